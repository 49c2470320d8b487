// Shared device primitives of the integer training kernels: the device error record, the rounding /
// bit-length / exp / isqrt arithmetic every kernel must reproduce exactly, lane-group reductions and
// the block quantiser.
//
// Arithmetic follows the reference's int64 specification (jatai_cuda/ops.py:34-89) evaluated in int32
// registers under the same invariant its CUDA library states (jatai_cuda/jatai_cuda.cu:3-9): every
// intermediate stays below 2^30, and a kernel that sees the invariant broken records a sentinel in the
// device error record instead of trapping.
#pragma once
#include <cstdint>
#include <cuda_runtime.h>

namespace jt {

constexpr int E_ZERO = -127;          // exponent of an all-zero block
constexpr int LIM = 1 << 30;          // register invariant |v| < 2^30
constexpr int SEM_TOPO = -100000;     // "block has no non-zero element"
constexpr int U_MIN = -2147483647;    // "-infinity" of scores / logits
constexpr unsigned FULL = 0xffffffffu;

// sentinel codes 1..6 are the reference's (jatai_cuda.cu:22); 7 is new: a bounded device-side wait ran out
enum { E_ACUM = 1, E_EXP = 2, E_SAT = 3, E_DIV = 4, E_SHL = 5, E_ARG = 6, E_TEMPO = 7 };

// Device error record (jatai_cuda.cu:24-28): the first event wins, n counts all of them.
struct Erro {
    int n, codigo, kid, pad;
    long long idx, valor, aux;
};
// The library is one translation unit (jatai_b200.cu includes every .cuh), so the record is defined here.
__device__ Erro g_erro;

// kept out of line: the error path is cold and must not bloat the hot loops
__device__ __noinline__ void reporta(int codigo, int kid, long long idx, long long valor, long long aux) {
    if (atomicAdd(&g_erro.n, 1) == 0) {
        g_erro.codigo = codigo; g_erro.kid = kid; g_erro.idx = idx; g_erro.valor = valor; g_erro.aux = aux;
        __threadfence();
    }
}

// ---------------------------------------------------------------------------------------- dependent launches
// Programmatic dependent launch: a kernel launched with the attribute may start while its predecessor in the stream is
// still draining; `pdl_espera` returns once the predecessor has completed and its writes are visible, so it goes before
// the first access to global memory (what comes before it - barrier set-up, tensor-memory allocation - overlaps the
// predecessor's tail).  `pdl_solta` would let the successor be scheduled as soon as every CTA of this grid has got that far
// instead of when they exit; measured, that is a loss (the waiting CTAs hold SMs the kernels of the other streams could
// use: 5.44 ms against 4.95 ms per 12-layer step), so it compiles to nothing unless JT_PDL_CEDO is defined.
// Without the attribute both are no-ops.
__device__ __forceinline__ void pdl_espera() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_solta() {
#ifdef JT_PDL_CEDO
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
#endif
}
// host: the switch (jt_pdl) and the launch of a kernel that contains pdl_espera
inline int& pdl_ligado() { static int v = 0; return v; }
template <typename... KP, typename... A>
static inline void lanca_pdl(void (*k)(KP...), dim3 grade, dim3 bloco, size_t smem, cudaStream_t st, A... a) {
    if (!pdl_ligado()) { k<<<grade, bloco, smem, st>>>(a...); return; }
    cudaLaunchConfig_t c = {};
    c.gridDim = grade; c.blockDim = bloco; c.dynamicSmemBytes = smem; c.stream = st;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    c.attrs = at; c.numAttrs = 1;
    (void)cudaLaunchKernelEx(&c, k, a...);                         // errors surface through cudaGetLastError like those of <<< >>>
}

// ---------------------------------------------------------------------------------------- arithmetic
__device__ __forceinline__ int bitlen(int x) { return 32 - __clz(x < 0 ? -x : x); }

// x * 2^-s for s >= 0, ties to even; |x| < 2^30 (ops.py:42-51 for s > 0).  s >= 31 gives 0.
__device__ __forceinline__ int rnd_d(int x, int s) {
    s = min(s, 31);
    if (s == 0) return x;
    return (x + ((1 << (s - 1)) - 1) + ((x >> s) & 1)) >> s;
}

// x * 2^-s for any sign of s; the left shift is reported (E_SHL) if it would leave the 2^30 range.
__device__ __forceinline__ int rnd(int x, int s, int kid, long long idx) {
    if (s > 0) return rnd_d(x, s);
    if (s == 0 || x == 0) return x;
    s = -s;
    if (s > 30 || bitlen(x) + s > 30) { reporta(E_SHL, kid, idx, x, -s); return 0; }
    return x << s;
}

// same, where the caller has proved that the left shift cannot lose bits
__device__ __forceinline__ int desloca(int x, int s) { return s >= 0 ? rnd_d(x, s) : x << min(-s, 31); }

// Q15 exp(-d/256), d >= 0 (ops.py:75-81)
__device__ __forceinline__ int exp_int(int d) {
    const int t = min(d, 6000) * 23637;
    const int n = t >> 22, f = (t & ((1 << 22) - 1)) >> 7;
    int p = -1295;
    p = ((p * f) >> 15) + 7556;
    p = ((p * f) >> 15) - 22645;
    p = ((p * f) >> 15) + 32765;
    return n > 30 ? 0 : p >> n;
}
// exp(-(mx - u)/256) with the difference clamped before subtracting (mx - u may not fit in int32)
__device__ __forceinline__ int exp_dif(int mx, int u) { return exp_int(u <= mx - 6000 ? 6000 : mx - u); }

// integer square root (ops.py:84-89: 10 Newton steps from a power of two above the root, each min(x, (x + n/x) >> 1); from
// above they converge to floor(sqrt(n)) well inside 10 steps for every n < 2^31, and the result is clamped to >= 1).
// Here: the fp32 estimate is within 1 of the root (n has at most 31 bits, the estimate's error is far below 1), two integer
// corrections make it exact.  r <= 46340, so r^2 and (r+1)^2 fit an unsigned 32-bit integer.
__device__ __forceinline__ int isqrt_i(int n) {
    n = max(n, 0);
    unsigned r = (unsigned)__float2int_rd(sqrtf((float)n));
    r = min(r, 46340u);
    if (r * r > (unsigned)n) r -= 1;
    if ((r + 1) * (r + 1) <= (unsigned)n) r += 1;
    return max((int)r, 1);
}

// ---------------------------------------------------------------------------------------- lane groups
// GL lanes (a power of two) at lane distance ST cooperate on one exponent block.  All 32 lanes must call.
// `mask` names the lanes that execute the call together (whole groups); FULL unless the caller has branched.
template <int GL, int ST = 1> __device__ __forceinline__ int grupo_max(int v, unsigned mask = FULL) {
#pragma unroll
    for (int o = GL / 2; o; o >>= 1) v = max(v, __shfl_xor_sync(mask, v, o * ST));
    return v;
}
template <int GL, int ST = 1> __device__ __forceinline__ int grupo_or(int v, unsigned mask = FULL) {
#pragma unroll
    for (int o = GL / 2; o; o >>= 1) v |= __shfl_xor_sync(mask, v, o * ST);
    return v;
}
__device__ __forceinline__ int warp_max(int v) { return grupo_max<32>(v); }
__device__ __forceinline__ int warp_sum(int v) {
#pragma unroll
    for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(FULL, v, o);
    return v;
}

// ---------------------------------------------------------------------------------------- 16-byte vectors
// A thread of the bandwidth kernels owns 16 consecutive elements: one 128-bit access of int8 data.
__device__ __forceinline__ void le16(const int8_t* p, int (&v)[16]) {
    const uint4 w = *reinterpret_cast<const uint4*>(p);
    const uint32_t u[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
    for (int i = 0; i < 4; i++) {
        v[4 * i + 0] = (int)(int8_t)(u[i] & 0xff);
        v[4 * i + 1] = (int)(int8_t)((u[i] >> 8) & 0xff);
        v[4 * i + 2] = (int)(int8_t)((u[i] >> 16) & 0xff);
        v[4 * i + 3] = (int)u[i] >> 24;
    }
}
__device__ __forceinline__ void desempacota16(const uint4& w, int (&v)[16]) {
    const uint32_t u[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
    for (int i = 0; i < 4; i++) {
        v[4 * i + 0] = (int)(int8_t)(u[i] & 0xff);
        v[4 * i + 1] = (int)(int8_t)((u[i] >> 8) & 0xff);
        v[4 * i + 2] = (int)(int8_t)((u[i] >> 16) & 0xff);
        v[4 * i + 3] = (int)u[i] >> 24;
    }
}
__device__ __forceinline__ uint32_t junta4(int a, int b, int c, int d) {
    return (uint32_t)(a & 0xff) | ((uint32_t)(b & 0xff) << 8) | ((uint32_t)(c & 0xff) << 16) | ((uint32_t)d << 24);
}
__device__ __forceinline__ void grava16(int8_t* p, const int (&q)[16]) {
    uint4 w;
    w.x = junta4(q[0], q[1], q[2], q[3]);
    w.y = junta4(q[4], q[5], q[6], q[7]);
    w.z = junta4(q[8], q[9], q[10], q[11]);
    w.w = junta4(q[12], q[13], q[14], q[15]);
    *reinterpret_cast<uint4*>(p) = w;
}
__device__ __forceinline__ void le16_i32(const int* p, int (&v)[16]) {
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const int4 w = reinterpret_cast<const int4*>(p)[i];
        v[4 * i] = w.x; v[4 * i + 1] = w.y; v[4 * i + 2] = w.z; v[4 * i + 3] = w.w;
    }
}
__device__ __forceinline__ void le16_i16(const int16_t* p, int (&v)[16]) {
#pragma unroll
    for (int i = 0; i < 2; i++) {
        const uint4 w = reinterpret_cast<const uint4*>(p)[i];
        const uint32_t u[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
        for (int j = 0; j < 4; j++) {
            v[8 * i + 2 * j] = (int)(int16_t)(u[j] & 0xffff);
            v[8 * i + 2 * j + 1] = (int)u[j] >> 16;
        }
    }
}

// ---------------------------------------------------------------------------------------- block quantiser
// ops.py:58-72.  Each of GL lanes holds NV values of one block.
//   top = max over non-zero values of e + bitlen(v);  E = top - 7;  q = rnd(v, E - e);
//   if any |q| > 127: E += 1 and round again;  E < -126 (or no non-zero value): zero block, E = -127.
// Returns E; q receives the mantissas (already inside +-127).

// all values share the exponent e: only the largest magnitude can overflow (rounding is monotone and odd)
template <int NV, int GL, int ST = 1>
__device__ __forceinline__ int quant_uniforme(const int (&v)[NV], int e, int (&q)[NV], int kid, long long idx0, unsigned mask = FULL) {
    int mx = 0;
#pragma unroll
    for (int i = 0; i < NV; i++) mx = max(mx, v[i] < 0 ? -v[i] : v[i]);
    mx = grupo_max<GL, ST>(mx, mask);
    if (mx >= LIM) reporta(E_ACUM, kid, idx0, mx, e);
    int sh = bitlen(mx) - 7;
    if (desloca(mx, sh) > 127) sh += 1;
    const int E = e + sh;
    if (mx == 0 || E < -126) {
#pragma unroll
        for (int i = 0; i < NV; i++) q[i] = 0;
        return E_ZERO;
    }
    if (E > 126) reporta(E_EXP, kid, idx0, E, e);
#pragma unroll
    for (int i = 0; i < NV; i++) q[i] = desloca(v[i], sh);
    return E;
}

// every value has its own exponent
template <int NV, int GL, int ST = 1>
__device__ __forceinline__ int quant_geral(const int (&v)[NV], const int (&e)[NV], int (&q)[NV], int kid, long long idx0, unsigned mask = FULL) {
    int topo = SEM_TOPO;
#pragma unroll
    for (int i = 0; i < NV; i++) {
        if (v[i] >= LIM || v[i] <= -LIM) reporta(E_ACUM, kid, idx0 + i, v[i], e[i]);
        if (v[i] != 0) topo = max(topo, e[i] + bitlen(v[i]));
    }
    topo = grupo_max<GL, ST>(topo, mask);
    // E >= e[i] + bitlen(v[i]) - 7, so a left shift moves v[i] up to 7 bits at most: it cannot lose bits
    int E = topo - 7, over = 0;
#pragma unroll
    for (int i = 0; i < NV; i++) {
        q[i] = desloca(v[i], E - e[i]);
        over |= (q[i] > 127) | (q[i] < -127);
    }
    if (grupo_or<GL, ST>(over, mask)) {
        E += 1;
#pragma unroll
        for (int i = 0; i < NV; i++) q[i] = desloca(v[i], E - e[i]);
    }
    if (topo == SEM_TOPO || E < -126) {
#pragma unroll
        for (int i = 0; i < NV; i++) q[i] = 0;
        return E_ZERO;
    }
    if (E > 126) reporta(E_EXP, kid, idx0, E, topo);
#pragma unroll
    for (int i = 0; i < NV; i++) {
        if (q[i] > 127 || q[i] < -127) reporta(E_SAT, kid, idx0 + i, q[i], E);
        q[i] = max(-127, min(127, q[i]));
    }
    return E;
}

// 16 int8 -> float without the conversion pipe: with its sign bit flipped a byte is b + 128 in 0..255; placed under the upper
// bytes of 1.5 * 2^23 it reads as the float 12582912 + 128 + b, and one subtraction leaves b exactly.
__device__ __forceinline__ void bytes_para_float(const uint4& r, float (&f)[16]) {
    const uint32_t u[4] = {r.x ^ 0x80808080u, r.y ^ 0x80808080u, r.z ^ 0x80808080u, r.w ^ 0x80808080u};
#pragma unroll
    for (int i = 0; i < 4; i++) {
        f[4 * i + 0] = __uint_as_float(__byte_perm(u[i], 0x4B400000u, 0x7650)) - 12583040.0f;
        f[4 * i + 1] = __uint_as_float(__byte_perm(u[i], 0x4B400000u, 0x7651)) - 12583040.0f;
        f[4 * i + 2] = __uint_as_float(__byte_perm(u[i], 0x4B400000u, 0x7652)) - 12583040.0f;
        f[4 * i + 3] = __uint_as_float(__byte_perm(u[i], 0x4B400000u, 0x7653)) - 12583040.0f;
    }
}

// Block quantiser in fp32 for integer-valued floats below 2^24 that share the exponent e (exact: ops.py:58-72).
// The largest magnitude gives bitlen through its exponent field; one FFMA against 1.5*2^23 rounds v * 2^-sh half
// to even (the low byte of the result's bit pattern is the mantissa); the "one more bit" retry is decided on the
// maximum alone, because rounding is monotone.  Returns E; `pac` receives the 16 mantissas.
template <int GL, int ST = 1>
__device__ __forceinline__ int quant_f32(const float (&f)[16], int e, uint4& pac, int kid, long long idx0, unsigned mask = FULL) {
    float mx = 0.f;
#pragma unroll
    for (int i = 0; i < 16; i++) mx = fmaxf(mx, fabsf(f[i]));
#pragma unroll
    for (int o = GL / 2; o; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(mask, mx, o * ST));
    const int expo = (__float_as_int(mx) >> 23) - 127;               // floor(log2 mx) for mx >= 1
    int sh = expo - 6;                                               // bitlen - 7
    float sc = __int_as_float((127 - sh) << 23);                     // 2^-sh
    if ((__float_as_int(fmaf(mx, sc, 12582912.0f)) & 0x1ff) > 127) { sh += 1; sc *= 0.5f; }
    const int E = e + sh;
    if (mx == 0.f || E < -126) { pac = make_uint4(0, 0, 0, 0); return E_ZERO; }
    if (E > 126) reporta(E_EXP, kid, idx0, E, e);
    uint32_t r[16];
#pragma unroll
    for (int i = 0; i < 16; i++) r[i] = (uint32_t)__float_as_int(fmaf(f[i], sc, 12582912.0f));
    pac.x = __byte_perm(__byte_perm(r[0], r[1], 0x0040), __byte_perm(r[2], r[3], 0x0040), 0x5410);
    pac.y = __byte_perm(__byte_perm(r[4], r[5], 0x0040), __byte_perm(r[6], r[7], 0x0040), 0x5410);
    pac.z = __byte_perm(__byte_perm(r[8], r[9], 0x0040), __byte_perm(r[10], r[11], 0x0040), 0x5410);
    pac.w = __byte_perm(__byte_perm(r[12], r[13], 0x0040), __byte_perm(r[14], r[15], 0x0040), 0x5410);
    return E;
}

}  // namespace jt
