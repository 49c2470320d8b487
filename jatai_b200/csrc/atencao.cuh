// Integer causal attention with ALiBi, forward and backward, for head dimension 4, 16 or 64 and T <= 1024.
//
// Specification: jatai_cuda/ops.py:186-258 (written there for head dimension 4), generalised as follows:
// the exponent of an element is the exponent of the block its column falls in, and a head is aligned to the
// maximum exponent over all tokens of the sequence and all columns of the head; 1/sqrt(hd) is the exact shift
// log2(hd)/2; the ALiBi slope exponent of head h stays the literal 8 - h/8 of the reference.
//
// Layouts (jatai_cuda/jatai_cuda.cu:827-838,858-867): QKV is one block tensor [Bt*T, 3D] (q | k | v), head h at
// columns h*hd..h*hd+hd-1 of each third; token row = b*T + t; P is uint8 [Bt*H][j][i] (key-major) with explicit
// zeros for j > i; outputs are raw (int32 + int16 exponent per element).
//
// Work decomposition: a CTA owns 32 query rows (or 32 keys in the column kernel of the backward) of one
// (sequence, head) and walks the other side in chunks of 128 rows staged, already aligned, in shared memory.
// Products run on the CUDA cores as 4x4 register tiles (aligned operands have 12 bits, so int8 tensor-core
// tiles would need digit splitting).  The backward needs two matrix-wide maxima per (sequence, head) between
// its phases (ops.py:235,244); they cross CTAs through atomicMax on a small workspace, and the per-row
// s_lin values through the same workspace:
//   k_ab1  max |gP| over j <= i                         (skipped by the upper-bound variant, which runs k_lim)
//   k_ab2  gP' = rnd(gP, sh); s_lin; max |dS| (and the maxima the upper-bound variant needs)
//   k_ab3q dS' = rnd(P (gP' - s_lin), sh2); gq = dS' . k          (row tiles)
//   k_ab3k dS' per key tile; gk = dS'^T . q, gv = P^T . dO   (no atomics on the outputs)
// When the workspace has room for a T x T int32 matrix per (sequence, head) (it stays in L2 at training sizes), gP is
// computed once and handed on: k_ab1 stores gP, k_ab2 turns it into gP', k_ab3q into dS', k_ab3k reads dS'.  Without
// it every phase recomputes dO . v^T from the operands.
#pragma once
#include "comum.cuh"

namespace jt {
namespace at {

constexpr int TI = 32, TJ = 128;
constexpr int N_EST = 8;            // ints of statistics per (sequence, head) in the workspace

__device__ __forceinline__ int incl_alibi(int h) { return max(8 - h / 8, 0); }

// max exponent of the head's columns [col0, col0 + HD) over the T rows of sequence b (all 256 threads call)
template <int HD>
__device__ __forceinline__ int max_cabeca(const int8_t* __restrict__ E, int ld_blocos, int blk, int linha0, int T, int col0, int* red, int tid) {
    const int nbh = HD > blk ? HD / blk : 1;
    int m = -128;
    for (int t = tid; t < T; t += 256) {
        const int8_t* p = E + (size_t)(linha0 + t) * ld_blocos + col0 / blk;
        for (int b = 0; b < nbh; b++) m = max(m, (int)p[b]);
    }
    m = warp_max(m);
    __syncthreads();
    if ((tid & 31) == 0) red[tid >> 5] = m;
    __syncthreads();
    int r = red[0];
#pragma unroll
    for (int i = 1; i < 8; i++) r = max(r, red[i]);
    return r;
}

// rows [linha0 + r0, +n) of one head, aligned to exponent emx with GA guard bits -> dst[r][HD+4] (int32);
// rows at or beyond `limite_linhas` (relative to linha0) are zero-filled.  ops.py:186-192
template <int HD>
__device__ __forceinline__ void carrega_alinhado(int* dst, const int8_t* __restrict__ m, const int8_t* __restrict__ E, int ld, int blk, int linha0,
                                                 int r0, int n, int limite_linhas, int col0, int emx, int GA, int tid) {
    constexpr int PK = HD + 4, VEC = HD >= 16 ? 16 : 4, PL = HD / VEC;
    const int ldb = ld / blk;
    for (int task = tid; task < n * PL; task += 256) {
        const int r = task / PL, c = (task % PL) * VEC;
        int* d = dst + r * PK + c;
        if (r0 + r >= limite_linhas) {
#pragma unroll
            for (int k = 0; k < VEC; k++) d[k] = 0;
            continue;
        }
        const size_t lin = (size_t)(linha0 + r0 + r);
        const int s = emx - (int)E[lin * ldb + (col0 + c) / blk];
        if (VEC == 16) {
            int v[16];
            le16(m + lin * ld + col0 + c, v);
#pragma unroll
            for (int k = 0; k < 16; k++) d[k] = rnd_d(v[k] << GA, s);
        } else {
            const uint32_t w = *reinterpret_cast<const uint32_t*>(m + lin * ld + col0 + c);
#pragma unroll
            for (int k = 0; k < 4; k++) d[k] = rnd_d(((int)(int8_t)(w >> (8 * k))) << GA, s);
        }
    }
}

// acc[r][c] = sum_d a_s[4 ty + r][d] * b_s[lane + 32 c][d]   (exact; |operands| <= 2032, hd <= 64)
// Only the first NC blocks of 32 rows of b_s are multiplied (the rest of acc stays 0): a causal row tile needs no
// product with the key blocks beyond its diagonal.
template <int HD, int NC>
__device__ __forceinline__ void prod4xn(const int* a_s, const int* b_s, int ty, int lane, int (&acc)[4][4]) {
    constexpr int PK = HD + 4;
#pragma unroll
    for (int d4 = 0; d4 < HD / 4; d4++) {
        int4 a[4], b[NC];
#pragma unroll
        for (int r = 0; r < 4; r++) a[r] = *reinterpret_cast<const int4*>(a_s + (4 * ty + r) * PK + 4 * d4);
#pragma unroll
        for (int c = 0; c < NC; c++) b[c] = *reinterpret_cast<const int4*>(b_s + (lane + 32 * c) * PK + 4 * d4);
#pragma unroll
        for (int r = 0; r < 4; r++)
#pragma unroll
            for (int c = 0; c < NC; c++) acc[r][c] += a[r].x * b[c].x + a[r].y * b[c].y + a[r].z * b[c].z + a[r].w * b[c].w;
    }
}
template <int HD>
__device__ __forceinline__ void prod4x4(const int* a_s, const int* b_s, int ty, int lane, int (&acc)[4][4], int nblocos = 4) {
#pragma unroll
    for (int r = 0; r < 4; r++)
#pragma unroll
        for (int c = 0; c < 4; c++) acc[r][c] = 0;
    if (nblocos >= 4) prod4xn<HD, 4>(a_s, b_s, ty, lane, acc);
    else if (nblocos == 3) prod4xn<HD, 3>(a_s, b_s, ty, lane, acc);
    else if (nblocos == 2) prod4xn<HD, 2>(a_s, b_s, ty, lane, acc);
    else prod4xn<HD, 1>(a_s, b_s, ty, lane, acc);
}

// Row products: out[r][d] = sum_j w_s[4 ty + r][j0 + j] * v_s[j][d] for the 4 rows of warp ty (P.V, dS'.k, dS'^T.q, P^T.dO).
// A lane owns 4 adjacent columns d (d4 = lane % (HD/4)) and one of NJ = 32 / (HD/4) interleaved groups of 4 keys, so
// both operands come in 128-bit shared-memory loads (4 rows x 4 keys of w, 4 keys x 4 columns of v -> 64 MACs per 8
// loads); the NJ partial sums are added with shuffles at the end (acumula4_fim).  WP (pitch of w_s) is a multiple of 4.
template <int HD>
__device__ __forceinline__ void acumula4(const int* w_s, int WP, const int* v_s, int j0, int nj, int ty, int lane, int (&acc)[4][4]) {
    constexpr int PK = HD + 4, ND4 = HD / 4, NJ = 32 / ND4;
    const int d4 = lane % ND4, jsub = lane / ND4;
    for (int jj = jsub * 4; jj < nj; jj += 4 * NJ) {
        int4 w[4], v[4];
#pragma unroll
        for (int r = 0; r < 4; r++) w[r] = *reinterpret_cast<const int4*>(w_s + (4 * ty + r) * WP + j0 + jj);
#pragma unroll
        for (int c = 0; c < 4; c++) v[c] = *reinterpret_cast<const int4*>(v_s + (jj + c) * PK + 4 * d4);
#pragma unroll
        for (int r = 0; r < 4; r++) {
            acc[r][0] += w[r].x * v[0].x + w[r].y * v[1].x + w[r].z * v[2].x + w[r].w * v[3].x;
            acc[r][1] += w[r].x * v[0].y + w[r].y * v[1].y + w[r].z * v[2].y + w[r].w * v[3].y;
            acc[r][2] += w[r].x * v[0].z + w[r].y * v[1].z + w[r].z * v[2].z + w[r].w * v[3].z;
            acc[r][3] += w[r].x * v[0].w + w[r].y * v[1].w + w[r].z * v[2].w + w[r].w * v[3].w;
        }
    }
}
// adds the NJ partial sums; afterwards the lanes with lane < HD/4 hold columns 4 lane .. 4 lane + 3 of the 4 rows
template <int HD>
__device__ __forceinline__ void acumula4_fim(int (&acc)[4][4]) {
    constexpr int ND4 = HD / 4;
#pragma unroll
    for (int o = 16; o >= ND4; o >>= 1)
#pragma unroll
        for (int r = 0; r < 4; r++)
#pragma unroll
            for (int k = 0; k < 4; k++) acc[r][k] += __shfl_xor_sync(FULL, acc[r][k], o);
}

// CTA-wide maximum of a non-negative per-thread value -> one atomicMax
__device__ __forceinline__ void max_cta_atomico(int v, int* destino, int* red, int tid) {
    v = warp_max(v);
    __syncthreads();
    if ((tid & 31) == 0) red[tid >> 5] = v;
    __syncthreads();
    if (tid == 0) {
        int r = red[0];
#pragma unroll
        for (int i = 1; i < 8; i++) r = max(r, red[i]);
        if (r > 0) atomicMax(destino, r);
    }
}

// -------------------------------------------------------------------------------------------------- forward
// ops.py:198-219.  grid (T/32, Bt*H), 256 threads.  Shared: u[32][T+4] int32, kv[128][hd+4], q[32][hd+4], pT[T][32] bytes.
template <int HD>
__global__ void __launch_bounds__(256) k_atencao(const int8_t* __restrict__ qm, const int8_t* __restrict__ qE, int* __restrict__ Oacc,
                                                 int16_t* __restrict__ Oe, uint8_t* __restrict__ P, int T, int H, int D, int GA, int blk, int lg2,
                                                 int kid) {
    constexpr int PK = HD + 4, ND4 = HD / 4;
    extern __shared__ __align__(16) int sm[];
    const int TP = T + 4;
    int* u_s = sm;
    int* kv_s = u_s + TI * TP;
    int* q_s = kv_s + TJ * PK;
    uint8_t* pT = reinterpret_cast<uint8_t*>(q_s + TI * PK);
    __shared__ int red[8];
    const int tid = threadIdx.x, ty = tid >> 5, lane = tid & 31;
    // causal work grows with the row tile: CTAs are dispatched in linear order, so the heaviest tiles of all heads go first
    const int ordem = blockIdx.y * gridDim.x + blockIdx.x;
    const int bh = ordem % gridDim.y, b = bh / H, h = bh % H, i0 = (gridDim.x - 1 - ordem / gridDim.y) * TI;
    const int ld = 3 * D, ldb = ld / blk, linha0 = b * T;
    const int emq = max_cabeca<HD>(qE, ldb, blk, linha0, T, h * HD, red, tid);
    const int emk = max_cabeca<HD>(qE, ldb, blk, linha0, T, D + h * HD, red, tid);
    const int emv = max_cabeca<HD>(qE, ldb, blk, linha0, T, 2 * D + h * HD, red, tid);
    const int s_u = -((emq - GA) + (emk - GA) - lg2 / 2 + 8);
    const int incl = incl_alibi(h);
    const int nproc = i0 + TI;                                         // keys this tile looks at: up to its diagonal (multiple of 32)
    carrega_alinhado<HD>(q_s, qm, qE, ld, blk, linha0, i0, TI, T, h * HD, emq, GA, tid);
    int mx[4] = {U_MIN, U_MIN, U_MIN, U_MIN};
    for (int j0 = 0; j0 < nproc; j0 += TJ) {
        __syncthreads();
        carrega_alinhado<HD>(kv_s, qm, qE, ld, blk, linha0, j0, min(TJ, i0 + TI - j0), T, D + h * HD, emk, GA, tid);     // keys up to the diagonal
        __syncthreads();
        int acc[4][4];
        prod4x4<HD>(q_s, kv_s, ty, lane, acc, (i0 + TI - j0 + 31) / 32);       // key blocks up to the diagonal
#pragma unroll
        for (int r = 0; r < 4; r++)
#pragma unroll
            for (int c = 0; c < 4; c++) {
                const int i = i0 + 4 * ty + r, j = j0 + lane + 32 * c;
                if (j >= nproc) continue;
                int u = U_MIN;
                if (j <= i) u = rnd(acc[r][c], s_u, kid, (long long)(linha0 + i) * D + h * HD) - ((i - j) << incl);
                u_s[(4 * ty + r) * TP + j] = u;
                mx[r] = max(mx[r], u);
            }
    }
    __syncthreads();
    // softmax of the 4 rows of this warp; P goes to u_s (ints, for P.V) and to pT (bytes, the stored layout)
#pragma unroll
    for (int r = 0; r < 4; r++) {
        const int i = i0 + 4 * ty + r, m = warp_max(mx[r]);
        int* ur = u_s + (4 * ty + r) * TP;
        int soma = 0;
        for (int j = lane; j < nproc; j += 32) {
            const int ex = j <= i ? exp_dif(m, ur[j]) >> 3 : 0;
            ur[j] = ex;
            soma += ex;
        }
        soma = warp_sum(soma);
        if (soma <= 0) { if (lane == 0) reporta(E_DIV, kid, (long long)(linha0 + i) * D + h * HD, soma, 0); soma = 1; }
        const int inv = (1 << 28) / soma;
        for (int j = lane; j < nproc; j += 32) {
            const int p = min((ur[j] * inv + (1 << 19)) >> 20, 255);
            ur[j] = p;
            pT[j * TI + 4 * ty + r] = (uint8_t)p;
        }
    }
    __syncthreads();
    // stored P: for every key j the 32 query rows of this tile are 32 contiguous bytes
    for (int k = tid; k < T * 2; k += 256) {
        const int j = k >> 1, hf = k & 1;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (j < nproc) v = *reinterpret_cast<const uint4*>(pT + j * TI + hf * 16);
        *reinterpret_cast<uint4*>(P + ((size_t)bh * T + j) * T + i0 + hf * 16) = v;
    }
    // O = P . V
    int o[4][4];
#pragma unroll
    for (int r = 0; r < 4; r++)
#pragma unroll
        for (int k = 0; k < 4; k++) o[r][k] = 0;
    for (int j0 = 0; j0 < nproc; j0 += TJ) {
        __syncthreads();
        carrega_alinhado<HD>(kv_s, qm, qE, ld, blk, linha0, j0, min(TJ, i0 + TI - j0), T, 2 * D + h * HD, emv, GA, tid);
        __syncthreads();
        acumula4<HD>(u_s, TP, kv_s, j0, min(TJ, i0 + TI - j0), ty, lane, o);     // P is zero beyond the diagonal
    }
    acumula4_fim<HD>(o);
    if (lane < ND4) {
        const int eo = (emv - GA) - 8;
        const uint32_t e2 = (uint32_t)(eo & 0xffff) | ((uint32_t)eo << 16);
#pragma unroll
        for (int r = 0; r < 4; r++) {
            const size_t p = (size_t)(linha0 + i0 + 4 * ty + r) * D + h * HD + 4 * lane;
            *reinterpret_cast<int4*>(Oacc + p) = make_int4(o[r][0], o[r][1], o[r][2], o[r][3]);
            *reinterpret_cast<uint2*>(Oe + p) = make_uint2(e2, e2);
        }
    }
}

// -------------------------------------------------------------------------------------------------- backward
struct ArgsTras {
    const int8_t* gom; const int8_t* goE; const int8_t* qm; const int8_t* qE; const uint8_t* P;
    int* Gacc; int16_t* Ge; int* est; int* sl;           // est: [Bt*H][N_EST]; sl: [Bt*H][T]
    int* mat;                                            // [Bt*H][T][T] (query-major) or nullptr: gP, then gP', then dS' handed from phase to phase
    int T, H, D, GA, blk, limite, kid;
};
// statistics slots
enum { S_GP = 0, S_DS = 1, S_P = 2, S_GPQ = 3, S_SL = 4, S_GO = 5, S_V1 = 6 };

__device__ __forceinline__ int desl1(const int* e, int limite) {
    return max(bitlen(limite ? e[S_GO] * e[S_V1] : e[S_GP]) - 15, 0);
}
__device__ __forceinline__ int desl2(const int* e, int limite) {
    return max(bitlen(limite ? e[S_P] * (e[S_GPQ] + e[S_SL]) : e[S_DS]) - 12, 0);
}

// upper-bound variant (ops.py:231-233): max_i ||dO_i||_inf and max_j ||v_j||_1 of the aligned operands.  grid Bt*H.
template <int HD>
__global__ void __launch_bounds__(256) k_lim(ArgsTras A) {
    __shared__ int red[8];
    const int tid = threadIdx.x, bh = blockIdx.x, b = bh / A.H, h = bh % A.H, T = A.T, D = A.D;
    const int linha0 = b * T;
    const int emg = max_cabeca<HD>(A.goE, D / A.blk, A.blk, linha0, T, h * HD, red, tid);
    const int emv = max_cabeca<HD>(A.qE, 3 * D / A.blk, A.blk, linha0, T, 2 * D + h * HD, red, tid);
    int mg = 0, mv = 0;
    for (int t = tid; t < T; t += 256) {
        const size_t lg = (size_t)(linha0 + t);
        int s1 = 0;
        for (int d = 0; d < HD; d++) {
            const int eg = A.goE[lg * (D / A.blk) + (h * HD + d) / A.blk], ev = A.qE[lg * (3 * D / A.blk) + (2 * D + h * HD + d) / A.blk];
            const int g = rnd_d((int)A.gom[lg * D + h * HD + d] << A.GA, emg - eg);
            const int v = rnd_d((int)A.qm[lg * 3 * D + 2 * D + h * HD + d] << A.GA, emv - ev);
            mg = max(mg, g < 0 ? -g : g);
            s1 += v < 0 ? -v : v;
        }
        mv = max(mv, s1);
    }
    max_cta_atomico(mg, A.est + bh * N_EST + S_GO, red, tid);
    max_cta_atomico(mv, A.est + bh * N_EST + S_V1, red, tid);
}

// FASE 1: max |gP| over j <= i.   FASE 2: gP', s_lin, maxima.   FASE 3: dS', gq.     grid (T/32, Bt*H)
template <int HD, int FASE>
__global__ void __launch_bounds__(256) k_ab_linhas(ArgsTras A) {
    constexpr int PK = HD + 4, ND4 = HD / 4;
    extern __shared__ __align__(16) int sm[];
    const int T = A.T, H = A.H, D = A.D, GA = A.GA, blk = A.blk, TP = T + 4;
    int* g_s = sm;                                  // [32][T+4]: gP', then dS'
    int* b_s = g_s + (FASE == 1 ? 0 : TI * TP);     // [128][PK]: v chunk, then k chunk
    int* a_s = b_s + TJ * PK;                       // [32][PK]: dO tile
    uint8_t* pT = reinterpret_cast<uint8_t*>(a_s + TI * PK);      // [T][32]
    __shared__ int red[8];
    __shared__ int sl_s[TI];
    const int tid = threadIdx.x, ty = tid >> 5, lane = tid & 31;
    const int ordem = blockIdx.y * gridDim.x + blockIdx.x;          // heaviest (last) row tiles of all heads first
    const int bh = ordem % gridDim.y, b = bh / H, h = bh % H, i0 = (gridDim.x - 1 - ordem / gridDim.y) * TI, linha0 = b * T;
    int* est = A.est + bh * N_EST;
    const int emg = max_cabeca<HD>(A.goE, D / blk, blk, linha0, T, h * HD, red, tid);
    const int emv = max_cabeca<HD>(A.qE, 3 * D / blk, blk, linha0, T, 2 * D + h * HD, red, tid);
    const int nproc = i0 + TI;                      // keys up to the diagonal of this row tile
    const int sh = FASE == 1 ? 0 : desl1(est, A.limite);
    int mgp = 0;
    // With the matrix workspace the product dO . v^T is computed once (phase 1, or phase 2 of the upper-bound variant):
    // phase 1 leaves gP there, phase 2 replaces it by gP', phase 3 by dS' for the key-tile kernel.
    int* mat = A.mat ? A.mat + ((size_t)bh * T + i0) * T : nullptr;                // rows i0.. of this (sequence, head)
    const bool le_mat = mat && (FASE == 3 || (FASE == 2 && !A.limite));
    if (le_mat) {
#pragma unroll
        for (int r4 = 0; r4 < 4; r4++) {
            const int r = 4 * ty + r4, i = i0 + r;
            for (int j = lane; j < nproc; j += 32) {
                int g = mat[(size_t)r * T + j];
                if (FASE == 2) {
                    g = j <= i ? rnd_d(g, sh) : 0;
                    mgp = max(mgp, g < 0 ? -g : g);
                }
                g_s[r * TP + j] = g;
            }
        }
    } else {
        carrega_alinhado<HD>(a_s, A.gom, A.goE, D, blk, linha0, i0, TI, T, h * HD, emg, GA, tid);
        for (int j0 = 0; j0 < nproc; j0 += TJ) {
            __syncthreads();
            carrega_alinhado<HD>(b_s, A.qm, A.qE, 3 * D, blk, linha0, j0, min(TJ, i0 + TI - j0), T, 2 * D + h * HD, emv, GA, tid);
            __syncthreads();
            int acc[4][4];
            prod4x4<HD>(a_s, b_s, ty, lane, acc, (i0 + TI - j0 + 31) / 32);
#pragma unroll
            for (int r = 0; r < 4; r++)
#pragma unroll
                for (int c = 0; c < 4; c++) {
                    const int i = i0 + 4 * ty + r, j = j0 + lane + 32 * c;
                    if (j >= nproc) continue;
                    if (FASE == 1 && mat) mat[(size_t)(4 * ty + r) * T + j] = acc[r][c];
                    const int g = j <= i ? rnd_d(acc[r][c], sh) : 0;
                    mgp = max(mgp, g < 0 ? -g : g);
                    if (FASE != 1) g_s[(4 * ty + r) * TP + j] = g;
                }
        }
    }
    if (FASE == 1) {
        max_cta_atomico(mgp, est + S_GP, red, tid);
        return;
    }
    // stored P of this tile: key-major, 32 bytes per key
    for (int k = tid; k < nproc * 2; k += 256) {
        const int j = k >> 1, hf = k & 1;
        *reinterpret_cast<uint4*>(pT + j * TI + hf * 16) = *reinterpret_cast<const uint4*>(A.P + ((size_t)bh * T + j) * T + i0 + hf * 16);
    }
    __syncthreads();
    if (FASE == 2) {
        int mds = 0, mp = 0, msl = 0;
#pragma unroll
        for (int r = 0; r < 4; r++) {
            const int* gr = g_s + (4 * ty + r) * TP;
            int s = 0;
            for (int j = lane; j < nproc; j += 32) s += (int)pT[j * TI + 4 * ty + r] * gr[j];
            s = warp_sum(s);
            const int sl = rnd_d(s, 8);
            if (lane == 0) A.sl[(size_t)bh * T + i0 + 4 * ty + r] = sl;
            msl = max(msl, sl < 0 ? -sl : sl);
            for (int j = lane; j < nproc; j += 32) {
                const int p = pT[j * TI + 4 * ty + r], ds = p * (gr[j] - sl);
                mds = max(mds, ds < 0 ? -ds : ds);
                mp = max(mp, p);
            }
        }
        if (mat)                                  // gP' of this tile for phase 3 and the key-tile kernel
#pragma unroll
            for (int r = 0; r < 4; r++)
                for (int j = lane; j < nproc; j += 32) mat[(size_t)(4 * ty + r) * T + j] = g_s[(4 * ty + r) * TP + j];
        max_cta_atomico(mds, est + S_DS, red, tid);
        if (A.limite) {
            max_cta_atomico(mp, est + S_P, red, tid);
            max_cta_atomico(mgp, est + S_GPQ, red, tid);
            max_cta_atomico(msl, est + S_SL, red, tid);
        }
        return;
    }
    // FASE 3
    const int sh2 = desl2(est, A.limite);
    if (tid < TI) sl_s[tid] = A.sl[(size_t)bh * T + i0 + tid];
    __syncthreads();
#pragma unroll
    for (int r = 0; r < 4; r++) {
        int* gr = g_s + (4 * ty + r) * TP;
        const int sl = sl_s[4 * ty + r];
        for (int j = lane; j < nproc; j += 32) {
            const int ds = rnd_d((int)pT[j * TI + 4 * ty + r] * (gr[j] - sl), sh2);
            gr[j] = ds;
            if (mat) mat[(size_t)(4 * ty + r) * T + j] = ds;
        }
    }
    const int emk = max_cabeca<HD>(A.qE, 3 * D / blk, blk, linha0, T, D + h * HD, red, tid);
    int o[4][4];
#pragma unroll
    for (int r = 0; r < 4; r++)
#pragma unroll
        for (int k = 0; k < 4; k++) o[r][k] = 0;
    for (int j0 = 0; j0 < nproc; j0 += TJ) {
        __syncthreads();
        carrega_alinhado<HD>(b_s, A.qm, A.qE, 3 * D, blk, linha0, j0, min(TJ, i0 + TI - j0), T, D + h * HD, emk, GA, tid);
        __syncthreads();
        acumula4<HD>(g_s, TP, b_s, j0, min(TJ, i0 + TI - j0), ty, lane, o);      // dS' is zero beyond the diagonal
    }
    acumula4_fim<HD>(o);
    if (lane < ND4) {
        const int eds = (emg - GA) + (emv - GA) + sh - 9 + sh2;
        const int e = eds + (emk - GA);
        const uint32_t e2 = (uint32_t)(e & 0xffff) | ((uint32_t)e << 16);
#pragma unroll
        for (int r = 0; r < 4; r++) {
            const size_t p = (size_t)(linha0 + i0 + 4 * ty + r) * 3 * D + h * HD + 4 * lane;
            *reinterpret_cast<int4*>(A.Gacc + p) = make_int4(o[r][0], o[r][1], o[r][2], o[r][3]);
            *reinterpret_cast<uint2*>(A.Ge + p) = make_uint2(e2, e2);
        }
    }
}

// key tiles: gk[j] = sum_i dS'[i][j] q[i], gv[j] = sum_i P[i][j] dO[i].   grid (T/32, Bt*H)
template <int HD>
__global__ void __launch_bounds__(256, 2) k_ab_colunas(ArgsTras A) {
    constexpr int PK = HD + 4, ND4 = HD / 4, CP = TJ + 4;
    extern __shared__ __align__(16) int sm[];
    const int T = A.T, H = A.H, D = A.D, GA = A.GA, blk = A.blk;
    int* a_s = sm;                    // [32][PK]  v tile (keys of this CTA)
    int* b_s = a_s + TI * PK;         // [128][PK] dO chunk
    int* c_s = b_s + TJ * PK;         // [128][PK] q chunk
    int* ds_c = c_s + TJ * PK;        // [32][132] dS' of the chunk
    int* p_c = ds_c + TI * CP;        // [32][132] P of the chunk
    __shared__ int red[8];
    const int tid = threadIdx.x, ty = tid >> 5, lane = tid & 31;
    const int ordem = blockIdx.y * gridDim.x + blockIdx.x;          // heaviest (first) key tiles of all heads first
    const int bh = ordem % gridDim.y, b = bh / H, h = bh % H, j0 = (ordem / gridDim.y) * TI, linha0 = b * T;
    const int* est = A.est + bh * N_EST;
    const int emg = max_cabeca<HD>(A.goE, D / blk, blk, linha0, T, h * HD, red, tid);
    const int emq = max_cabeca<HD>(A.qE, 3 * D / blk, blk, linha0, T, h * HD, red, tid);
    const int emv = max_cabeca<HD>(A.qE, 3 * D / blk, blk, linha0, T, 2 * D + h * HD, red, tid);
    const int sh = desl1(est, A.limite), sh2 = desl2(est, A.limite);
    const int* mat = A.mat ? A.mat + (size_t)bh * T * T : nullptr;       // dS' left by phase 3, [i][j]
    if (!mat) carrega_alinhado<HD>(a_s, A.qm, A.qE, 3 * D, blk, linha0, j0, TI, T, 2 * D + h * HD, emv, GA, tid);
    int gk[4][4], gv[4][4];
#pragma unroll
    for (int r = 0; r < 4; r++)
#pragma unroll
        for (int k = 0; k < 4; k++) gk[r][k] = gv[r][k] = 0;
    for (int ic = (j0 / TJ) * TJ; ic < T; ic += TJ) {
        __syncthreads();
        const int antes = mat ? max(j0 - ic, 0) : 0;          // query rows before the key tile are not needed (the recomputing path reads them)
        carrega_alinhado<HD>(b_s + antes * PK, A.gom, A.goE, D, blk, linha0, ic + antes, TJ - antes, T, h * HD, emg, GA, tid);
        carrega_alinhado<HD>(c_s + antes * PK, A.qm, A.qE, 3 * D, blk, linha0, ic + antes, TJ - antes, T, h * HD, emq, GA, tid);
        __syncthreads();
        if (mat) {
            // dS' of the chunk from the workspace: a warp reads the 32 keys of one query row (128 contiguous bytes)
            for (int il = ty; il < TJ; il += 8) {
                const int i = ic + il, j = j0 + lane;
                ds_c[lane * CP + il] = (i < T && i >= j) ? mat[(size_t)i * T + j] : 0;
            }
#pragma unroll
            for (int r = 0; r < 4; r++)
#pragma unroll
                for (int c = 0; c < 4; c++) {
                    const int j = j0 + 4 * ty + r, il = lane + 32 * c, i = ic + il;
                    p_c[(4 * ty + r) * CP + il] = (i < T && i >= j) ? (int)A.P[((size_t)bh * T + j) * T + i] : 0;
                }
        } else {
            int acc[4][4];
            prod4x4<HD>(a_s, b_s, ty, lane, acc);      // acc[r][c] = gP[i = ic + lane + 32 c][j = j0 + 4 ty + r]
#pragma unroll
            for (int r = 0; r < 4; r++)
#pragma unroll
                for (int c = 0; c < 4; c++) {
                    const int j = j0 + 4 * ty + r, il = lane + 32 * c, i = ic + il;
                    int p = 0, ds = 0;
                    if (i < T && i >= j) {
                        p = A.P[((size_t)bh * T + j) * T + i];
                        ds = rnd_d(p * (rnd_d(acc[r][c], sh) - A.sl[(size_t)bh * T + i]), sh2);
                    }
                    ds_c[(4 * ty + r) * CP + il] = ds;
                    p_c[(4 * ty + r) * CP + il] = p;
                }
        }
        __syncthreads();
        const int ni = min(TJ, T - ic), pula = max(j0 - ic, 0);       // queries before the key tile see none of its keys
        acumula4<HD>(ds_c, CP, c_s + pula * PK, pula, ni - pula, ty, lane, gk);
        acumula4<HD>(p_c, CP, b_s + pula * PK, pula, ni - pula, ty, lane, gv);
    }
    acumula4_fim<HD>(gk);
    acumula4_fim<HD>(gv);
    if (lane < ND4) {
        const int ego = emg - GA, eds = ego + (emv - GA) + sh - 9 + sh2;
        const int e_k = eds + (emq - GA), e_v = ego - 8;
        const uint32_t k2 = (uint32_t)(e_k & 0xffff) | ((uint32_t)e_k << 16), v2 = (uint32_t)(e_v & 0xffff) | ((uint32_t)e_v << 16);
#pragma unroll
        for (int r = 0; r < 4; r++) {
            const size_t p = (size_t)(linha0 + j0 + 4 * ty + r) * 3 * D + D + h * HD + 4 * lane;
            *reinterpret_cast<int4*>(A.Gacc + p) = make_int4(gk[r][0], gk[r][1], gk[r][2], gk[r][3]);
            *reinterpret_cast<uint2*>(A.Ge + p) = make_uint2(k2, k2);
            *reinterpret_cast<int4*>(A.Gacc + p + D) = make_int4(gv[r][0], gv[r][1], gv[r][2], gv[r][3]);
            *reinterpret_cast<uint2*>(A.Ge + p + D) = make_uint2(v2, v2);
        }
    }
}

inline size_t smem_frente(int HD, int T) { return 4 * ((size_t)TI * (T + 4) + TJ * (HD + 4) + TI * (HD + 4)) + (size_t)T * TI; }
inline size_t smem_linhas(int HD, int T, int fase) {
    return 4 * ((fase == 1 ? 0 : (size_t)TI * (T + 4)) + TJ * (HD + 4) + TI * (HD + 4)) + (size_t)T * TI;
}
inline size_t smem_colunas(int HD) { return 4 * ((size_t)TI * (HD + 4) + 2 * TJ * (HD + 4) + 2 * TI * (TJ + 4)); }

}  // namespace at

// Workspace of the attention backward (statistics, s_lin, the T x T matrices), one per device, grown on demand.
// A superseded buffer is never freed: a CUDA graph recorded earlier may still hold its address.  Growth needs
// cudaMalloc, which a stream capture does not allow: a call that would have to grow while its stream is capturing is
// refused (cudaErrorStreamCaptureUnsupported); run one step eagerly before capturing, as the reference's loop does.
constexpr int AT_MAX_DEV = 64;
static void* g_at_ws[AT_MAX_DEV];
static size_t g_at_ws_bytes[AT_MAX_DEV];

// the current device's workspace, at least `bytes` long (0 = ok, else a cudaError_t)
static int at_ws(size_t bytes, cudaStream_t st, void** p) {
    int dev = 0;
    cudaError_t c = cudaGetDevice(&dev);
    if (c != cudaSuccess) return (int)c;
    if (dev < 0 || dev >= AT_MAX_DEV) return (int)cudaErrorInvalidDevice;
    if (bytes > g_at_ws_bytes[dev]) {
        cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
        if (cudaStreamIsCapturing(st, &cap) != cudaSuccess || cap != cudaStreamCaptureStatusNone) return (int)cudaErrorStreamCaptureUnsupported;
        void* novo = nullptr;
        c = cudaMalloc(&novo, bytes);
        if (c != cudaSuccess) return (int)c;
        g_at_ws[dev] = novo;              // the old buffer stays allocated until the process exits
        g_at_ws_bytes[dev] = bytes;
    }
    *p = g_at_ws[dev];
    return 0;
}

static int at_log2(int x) { int k = 0; while ((1 << k) < x) k++; return (1 << k) == x ? k : -1; }

// raises a kernel's dynamic shared-memory limit; remembered per kernel, so a repeated launch makes no runtime call
static cudaError_t at_smem_ptr(const void* kern, size_t bytes) {
    static const void* quem[64];
    static int onde[64];                  // the attribute belongs to (kernel, device)
    static size_t quanto[64];
    static int n = 0;
    int dev = 0;
    cudaError_t c = cudaGetDevice(&dev);
    if (c != cudaSuccess) return c;
    int i = 0;
    while (i < n && !(quem[i] == kern && onde[i] == dev)) i++;
    if (i < n && bytes <= quanto[i]) return cudaSuccess;
    c = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
    if (c != cudaSuccess) return c;
    if (i == n && n < 64) { quem[n] = kern; onde[n] = dev; n++; }
    if (i < 64) quanto[i] = bytes;
    return cudaSuccess;
}
template <typename K>
static cudaError_t at_smem(K kern, size_t bytes) { return at_smem_ptr(reinterpret_cast<const void*>(kern), bytes); }

static bool at_valido(int blk, int Bt, int T, int H, int D, int* hd, int* lg2) {
    if (Bt <= 0 || T <= 0 || H <= 0 || D <= 0 || D % H) return false;
    *hd = D / H;
    *lg2 = at_log2(*hd);
    if (!(*hd == 4 || *hd == 16 || *hd == 64)) return false;
    if (T % 32 || T > 1024 || D % blk || (3 * D) % blk) return false;
    if (*hd < blk ? blk % *hd : *hd % blk) return false;
    return true;
}

static int atencao_frente(int blk, const int8_t* qm, const int8_t* qE, int* Oacc, int16_t* Oe, uint8_t* P, int Bt, int T, int H, int D, int GA,
                          int kid, cudaStream_t st) {
    int hd, lg2;
    if (!at_valido(blk, Bt, T, H, D, &hd, &lg2)) return (int)cudaErrorInvalidValue;
    const dim3 grade(T / at::TI, Bt * H);
    const size_t sm = at::smem_frente(hd, T);
    cudaError_t c;
#define JT_F(HD)                                                                                              \
    if ((c = at_smem(at::k_atencao<HD>, sm)) != cudaSuccess) return (int)c;                                    \
    at::k_atencao<HD><<<grade, 256, sm, st>>>(qm, qE, Oacc, Oe, P, T, H, D, GA, blk, lg2, kid);
    if (hd == 4) { JT_F(4) } else if (hd == 16) { JT_F(16) } else { JT_F(64) }
#undef JT_F
    return (int)cudaGetLastError();
}

static int atencao_tras_ws(int blk, const int8_t* gom, const int8_t* goE, const int8_t* qm, const int8_t* qE, const uint8_t* P, int* Gacc,
                           int16_t* Ge, int Bt, int T, int H, int D, int GA, int limite, int kid, cudaStream_t st, int* ws, bool com_matriz) {
    int hd, lg2;
    if (!at_valido(blk, Bt, T, H, D, &hd, &lg2)) return (int)cudaErrorInvalidValue;
    const int BH = Bt * H;
    at::ArgsTras A = {gom, goE, qm, qE, P, Gacc, Ge, ws, ws + (size_t)BH * at::N_EST, com_matriz ? ws + (size_t)BH * (at::N_EST + T) : nullptr,
                      T, H, D, GA, blk, limite, kid};
    cudaError_t c = cudaMemsetAsync(ws, 0, (size_t)BH * at::N_EST * sizeof(int), st);
    if (c != cudaSuccess) return (int)c;
    const dim3 grade(T / at::TI, BH);
#define JT_B(HD)                                                                                                          \
    {                                                                                                                     \
        if (limite) at::k_lim<HD><<<BH, 256, 0, st>>>(A);                                                                 \
        else {                                                                                                            \
            if ((c = at_smem(at::k_ab_linhas<HD, 1>, at::smem_linhas(HD, T, 1))) != cudaSuccess) return (int)c;             \
            at::k_ab_linhas<HD, 1><<<grade, 256, at::smem_linhas(HD, T, 1), st>>>(A);                                     \
        }                                                                                                                 \
        if ((c = at_smem(at::k_ab_linhas<HD, 2>, at::smem_linhas(HD, T, 2))) != cudaSuccess) return (int)c;                 \
        at::k_ab_linhas<HD, 2><<<grade, 256, at::smem_linhas(HD, T, 2), st>>>(A);                                         \
        if ((c = at_smem(at::k_ab_linhas<HD, 3>, at::smem_linhas(HD, T, 3))) != cudaSuccess) return (int)c;                 \
        at::k_ab_linhas<HD, 3><<<grade, 256, at::smem_linhas(HD, T, 3), st>>>(A);                                         \
        if ((c = at_smem(at::k_ab_colunas<HD>, at::smem_colunas(HD))) != cudaSuccess) return (int)c;                        \
        at::k_ab_colunas<HD><<<grade, 256, at::smem_colunas(HD), st>>>(A);                                                \
    }
    if (hd == 4) JT_B(4) else if (hd == 16) JT_B(16) else JT_B(64)
#undef JT_B
    return (int)cudaGetLastError();
}

static int atencao_tras(int blk, const int8_t* gom, const int8_t* goE, const int8_t* qm, const int8_t* qE, const uint8_t* P, int* Gacc,
                        int16_t* Ge, int Bt, int T, int H, int D, int GA, int limite, int kid, cudaStream_t st) {
    if (Bt <= 0 || T <= 0 || H <= 0) return (int)cudaErrorInvalidValue;
    // statistics and s_lin, plus the T x T matrix per (sequence, head) that carries gP / gP' / dS' between the phases
    // (1 GiB at most; beyond that the phases recompute instead)
    const size_t base = (size_t)Bt * H * (at::N_EST + T), matriz = (size_t)Bt * H * T * T;
    const bool com_matriz = matriz <= ((size_t)1 << 28);
    const size_t precisa = base + (com_matriz ? matriz : 0);
    int* ws = nullptr;
    if (int r = at_ws(precisa * sizeof(int), st, reinterpret_cast<void**>(&ws))) return r;
    return atencao_tras_ws(blk, gom, goE, qm, qE, P, Gacc, Ge, Bt, T, H, D, GA, limite, kid, st, ws, com_matriz);
}

}  // namespace jt
