/* TEST INFRASTRUCTURE - plain C restatement of the reference's block GEMM specification.
 *
 * Follows jatai_cuda/ops.py:95-108 (OpsRef.gemm) and ops.py:42-51,58-72 (rnd, quant) of the reference,
 * with the block length as a parameter.  Used by tests/ as a fast checker at sizes where the torch int64
 * spec is slow, and by bench.py as the timed CPU baseline (OpenMP over output rows).  Never linked or
 * called by the library in jatai_b200/.
 *
 * Build: gcc -O3 -march=x86-64-v3 -pthread -shared -fPIC gemm_ref.c -o liboracle_gemm.so
 */
#include <pthread.h>
#include <stdint.h>
#include <stdlib.h>
#include <unistd.h>

#define E_ZERO (-127)
#define GG 4

static inline int bitlen64(int64_t x) {
    uint64_t a = x < 0 ? (uint64_t)(-x) : (uint64_t)x;
    return a ? 64 - __builtin_clzll(a) : 0;
}

/* x * 2^-s, ties to even; s <= 0 shifts left (ops.py:42-51) */
static inline int64_t rnd64(int64_t x, int s) {
    if (s <= 0) {
        int l = -s > 62 ? 62 : -s;
        return (int64_t)((uint64_t)x << l);
    }
    if (s > 62) s = 62;
    int64_t fl = x >> s;
    int64_t rem = x - (int64_t)((uint64_t)fl << s);
    int64_t half = (int64_t)1 << (s - 1);
    if (rem > half || (rem == half && (fl & 1))) fl++;
    return fl;
}

/* one block of `blk` values sharing (per element) exponents e[] -> int8 mantissas + exponent (ops.py:58-72) */
static void quant_bloco(const int64_t* v, const int64_t* e, int blk, int8_t* m, int8_t* Eo) {
    int64_t top = INT64_MIN;
    for (int i = 0; i < blk; i++)
        if (v[i] != 0) { int64_t t = e[i] + bitlen64(v[i]); if (t > top) top = t; }
    if (top == INT64_MIN) { for (int i = 0; i < blk; i++) m[i] = 0; *Eo = E_ZERO; return; }
    int64_t E = top - 7;
    int over = 0;
    for (int i = 0; i < blk; i++) { int64_t q = rnd64(v[i], (int)(E - e[i])); if (q > 127 || q < -127) over = 1; }
    E += over;
    if (E < -126) { for (int i = 0; i < blk; i++) m[i] = 0; *Eo = E_ZERO; return; }
    for (int i = 0; i < blk; i++) {
        int64_t q = rnd64(v[i], (int)(E - e[i]));
        m[i] = (int8_t)(q > 127 ? 127 : q < -127 ? -127 : q);
    }
    *Eo = (int8_t)E;
}

typedef struct {
    const int8_t *A, *EA, *B, *EB, *RAo;
    const int* RB;
    int N, K, blk, m1;
    int32_t* acc; int16_t* e; int8_t* Cm; int8_t* CE;
    int* next;                       /* shared row counter, advanced atomically 4 rows at a time */
} Job;

static void* worker(void* arg) {
    const Job* J = (const Job*)arg;
    const int N = J->N, K = J->K, blk = J->blk, nb = K / blk;
    int64_t* row = (int64_t*)malloc(sizeof(int64_t) * (size_t)N);
    int64_t* er = (int64_t*)malloc(sizeof(int64_t) * (size_t)N);
    for (;;) {
        int i0 = __atomic_fetch_add(J->next, 4, __ATOMIC_RELAXED);
        if (i0 >= J->m1) break;
        for (int i = i0; i < i0 + 4 && i < J->m1; i++) {
            int RA = -128;
            if (J->RAo) RA = J->RAo[i];
            else for (int b = 0; b < nb; b++) if (J->EA[(size_t)i * nb + b] > RA) RA = J->EA[(size_t)i * nb + b];
            const int8_t* a = J->A + (size_t)i * K;
            for (int j = 0; j < N; j++) {
                const int8_t* bb = J->B + (size_t)j * K;
                int64_t s64 = 0;
                for (int b = 0; b < nb; b++) {
                    int32_t p = 0;
                    const int8_t* ap = a + b * blk;
                    const int8_t* bp = bb + b * blk;
                    for (int k = 0; k < blk; k++) p += (int32_t)ap[k] * (int32_t)bp[k];
                    int s = (RA - J->EA[(size_t)i * nb + b]) + (J->RB[j] - J->EB[(size_t)j * nb + b]);
                    s64 += rnd64((int64_t)p << GG, s);
                }
                row[j] = s64;
                er[j] = (int64_t)RA + J->RB[j] - GG;
            }
            if (J->acc) for (int j = 0; j < N; j++) {
                J->acc[(size_t)i * N + j] = (int32_t)row[j];
                int64_t ee = er[j] < -30000 ? -30000 : er[j];
                J->e[(size_t)i * N + j] = (int16_t)ee;
            }
            if (J->Cm) for (int g = 0; g < N / blk; g++)
                quant_bloco(row + g * blk, er + g * blk, blk, J->Cm + (size_t)i * N + g * blk, J->CE + (size_t)i * (N / blk) + g);
        }
    }
    free(row); free(er);
    return NULL;
}

int oracle_threads(void) {
    long n = sysconf(_SC_NPROCESSORS_ONLN);
    const char* lim = getenv("ORACLE_THREADS");
    if (lim && atoi(lim) > 0) n = atoi(lim);
    return n < 1 ? 1 : n > 256 ? 256 : (int)n;
}

/* C[M,N] = A[M,K] . B[N,K]^T, both operands blocked along K.
 * RAo/RBo: optional externally supplied row-maximum exponents (data-parallel ranks pass the global maxima).
 * Outputs (each may be NULL): acc/e raw (int32 + int16 per element), Cm/CE block output along N.
 * Only rows [m0, m1) are computed, so a caller can time or check a slab.  Threads: one per online core
 * (ORACLE_THREADS overrides), rows handed out dynamically. */
int oracle_gemm(const int8_t* A, const int8_t* EA, const int8_t* B, const int8_t* EB, int M, int N, int K, int blk,
                const int8_t* RAo, const int8_t* RBo, int32_t* acc, int16_t* e, int8_t* Cm, int8_t* CE, int m0, int m1) {
    if (K % blk || N % blk || m0 < 0 || m1 > M) return 1;
    const int nb = K / blk;
    int* RB = (int*)malloc(sizeof(int) * (size_t)N);
    for (int j = 0; j < N; j++) {
        int r = -128;
        if (RBo) r = RBo[j];
        else for (int b = 0; b < nb; b++) if (EB[(size_t)j * nb + b] > r) r = EB[(size_t)j * nb + b];
        RB[j] = r;
    }
    int next = m0;
    Job J = {A, EA, B, EB, RAo, RB, N, K, blk, m1, acc, e, Cm, CE, &next};
    int nt = oracle_threads();
    pthread_t th[256];
    for (int t = 1; t < nt; t++) pthread_create(&th[t], NULL, worker, &J);
    worker(&J);
    for (int t = 1; t < nt; t++) pthread_join(th[t], NULL);
    free(RB);
    return 0;
}
