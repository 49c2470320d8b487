// Integer causal attention for short sequences (T <= 128) and small heads (head dimension 4 or 16): one CTA per (sequence,
// head), one thread per token.  This is the shape of the reference's own model (64 heads of 4, T = 128), where a head's whole
// problem - 128 x 128 scores over a 4-wide contraction - is too small to tile: the tiled kernels of atencao.cuh spend their time
// in launches, tile set-up and the cross-CTA maxima of the backward.  Here the operands of a head live in shared memory, a thread
// walks its query row (or, in the last pass of the backward, its key column), the two matrix-wide maxima of the backward are
// CTA-level reductions, and forward and backward are one launch each.  Scores are recomputed in every pass instead of stored.
//
// Specification and layouts as in atencao.cuh (jatai_cuda/ops.py:186-258; jatai_cuda/jatai_cuda.cu:822-1006): QKV [Bt*T, 3D]
// block tensor, P uint8 [Bt*H][j][i] with explicit zeros for j > i, raw outputs.
#pragma once
#include "comum.cuh"
#include "atencao.cuh"

namespace jt {
namespace atp {

constexpr int TMAX = 128;

// CTA-wide maximum of a per-thread value (blockDim.x = multiple of 32, <= 128); every thread gets the result
__device__ __forceinline__ int max_cta(int v, int* red, int tid) {
    v = warp_max(v);
    __syncthreads();
    if ((tid & 31) == 0) red[tid >> 5] = v;
    __syncthreads();
    int r = red[0];
    for (int w = 1; w < (int)(blockDim.x >> 5); w++) r = max(r, red[w]);
    return r;
}

// row `lin` of one head (HD columns from col0), aligned to exponent emx with GA guard bits (ops.py:186-192)
template <int HD>
__device__ __forceinline__ void linha_alinhada(const int8_t* __restrict__ m, const int8_t* __restrict__ E, size_t lin, int ld, int blk, int col0, int emx,
                                               int GA, int (&v)[HD]) {
    const int s = emx - (int)E[lin * (ld / blk) + col0 / blk];
    if (HD == 4) {
        const uint32_t w = *reinterpret_cast<const uint32_t*>(m + lin * ld + col0);
#pragma unroll
        for (int k = 0; k < 4; k++) v[k] = rnd_d(((int)(int8_t)(w >> (8 * k))) << GA, s);
    } else {
        int t[16];
        le16(m + lin * ld + col0, t);
#pragma unroll
        for (int k = 0; k < HD; k++) v[k] = rnd_d(t[k] << GA, s);
    }
}
template <int HD>
__device__ __forceinline__ int ponto(const int (&a)[HD], const int* __restrict__ b) {
    int s = 0;
#pragma unroll
    for (int k4 = 0; k4 < HD / 4; k4++) {
        const int4 w = reinterpret_cast<const int4*>(b)[k4];
        s += a[4 * k4] * w.x + a[4 * k4 + 1] * w.y + a[4 * k4 + 2] * w.z + a[4 * k4 + 3] * w.w;
    }
    return s;
}
template <int HD>
__device__ __forceinline__ void guarda(int* dst, const int (&v)[HD]) {
#pragma unroll
    for (int k4 = 0; k4 < HD / 4; k4++) reinterpret_cast<int4*>(dst)[k4] = make_int4(v[4 * k4], v[4 * k4 + 1], v[4 * k4 + 2], v[4 * k4 + 3]);
}
template <int HD>
__device__ __forceinline__ void grava_cru(int* acc, int16_t* e, size_t p, const int (&o)[HD], int ex) {
    const uint32_t e2 = (uint32_t)(ex & 0xffff) | ((uint32_t)ex << 16);
#pragma unroll
    for (int k4 = 0; k4 < HD / 4; k4++) {
        *reinterpret_cast<int4*>(acc + p + 4 * k4) = make_int4(o[4 * k4], o[4 * k4 + 1], o[4 * k4 + 2], o[4 * k4 + 3]);
        *reinterpret_cast<uint2*>(e + p + 4 * k4) = make_uint2(e2, e2);
    }
}

// -------------------------------------------------------------------------------------------------- forward
// ops.py:198-219.  grid Bt*H, T threads (thread = query row).  Three passes over the keys j <= i: row maximum, sum of the
// exponentials, then P (stored key-major, so the threads of a warp write consecutive bytes) and O = P . V.
template <int HD>
__global__ void __launch_bounds__(TMAX) k_atencao_peq(const int8_t* __restrict__ qm, const int8_t* __restrict__ qE, int* __restrict__ Oacc,
                                                      int16_t* __restrict__ Oe, uint8_t* __restrict__ P, int T, int H, int D, int GA, int blk, int lg2,
                                                      int kid) {
    __shared__ __align__(16) int k_s[TMAX * HD];
    __shared__ __align__(16) int v_s[TMAX * HD];
    __shared__ int red[4];
    const int i = threadIdx.x, bh = blockIdx.x, b = bh / H, h = bh % H, linha0 = b * T, ld = 3 * D, ldb = ld / blk;
    const size_t lin = (size_t)(linha0 + i);
    const int emq = max_cta((int)qE[lin * ldb + (h * HD) / blk], red, i);
    const int emk = max_cta((int)qE[lin * ldb + (D + h * HD) / blk], red, i);
    const int emv = max_cta((int)qE[lin * ldb + (2 * D + h * HD) / blk], red, i);
    int q[HD], t[HD];
    linha_alinhada<HD>(qm, qE, lin, ld, blk, h * HD, emq, GA, q);
    linha_alinhada<HD>(qm, qE, lin, ld, blk, D + h * HD, emk, GA, t);
    guarda<HD>(k_s + i * HD, t);
    linha_alinhada<HD>(qm, qE, lin, ld, blk, 2 * D + h * HD, emv, GA, t);
    guarda<HD>(v_s + i * HD, t);
    __syncthreads();
    const int s_u = -((emq - GA) + (emk - GA) - lg2 / 2 + 8), incl = at::incl_alibi(h);
    const long long idx = (long long)lin * D + h * HD;
    auto score = [&](int j) { return rnd(ponto<HD>(q, k_s + j * HD), s_u, kid, idx) - ((i - j) << incl); };
    int m = U_MIN;
    for (int j = 0; j <= i; j++) m = max(m, score(j));
    int soma = 0;
    for (int j = 0; j <= i; j++) soma += exp_dif(m, score(j)) >> 3;
    if (soma <= 0) { reporta(E_DIV, kid, idx, soma, 0); soma = 1; }
    const int inv = (1 << 28) / soma;
    int o[HD];
#pragma unroll
    for (int k = 0; k < HD; k++) o[k] = 0;
    uint8_t* Pc = P + (size_t)bh * T * T + i;
    for (int j = 0; j < T; j++) {                                  // every thread of the warp stores its byte of key row j
        int p = 0;
        if (j <= i) {
            p = min(((exp_dif(m, score(j)) >> 3) * inv + (1 << 19)) >> 20, 255);
            const int* vj = v_s + j * HD;
#pragma unroll
            for (int k4 = 0; k4 < HD / 4; k4++) {
                const int4 w = reinterpret_cast<const int4*>(vj)[k4];
                o[4 * k4] += p * w.x; o[4 * k4 + 1] += p * w.y; o[4 * k4 + 2] += p * w.z; o[4 * k4 + 3] += p * w.w;
            }
        }
        Pc[(size_t)j * T] = (uint8_t)p;
    }
    grava_cru<HD>(Oacc, Oe, (size_t)lin * D + h * HD, o, (emv - GA) - 8);
}

// -------------------------------------------------------------------------------------------------- backward
// ops.py:221-258.  grid Bt*H, T threads.  Passes (thread = query row unless stated): max |gP| (or, upper-bound variant, the operand
// norms); s_lin and max |dS|; dS' and gq; then thread = key column: gk and gv.  P of the head sits in shared memory.
template <int HD>
__global__ void __launch_bounds__(TMAX) k_atencao_back_peq(const int8_t* __restrict__ gom, const int8_t* __restrict__ goE, const int8_t* __restrict__ qm,
                                                           const int8_t* __restrict__ qE, const uint8_t* __restrict__ P, int* __restrict__ Gacc,
                                                           int16_t* __restrict__ Ge, int T, int H, int D, int GA, int blk, int limite, int kid) {
    extern __shared__ __align__(16) int sm[];
    int* q_s = sm;                     // [T][HD] each
    int* k_s = q_s + T * HD;
    int* v_s = k_s + T * HD;
    int* g_s = v_s + T * HD;
    int* sl_s = g_s + T * HD;          // [T]
    uint8_t* P_s = reinterpret_cast<uint8_t*>(sl_s + T);      // [T][T + 4]: row = key j
    __shared__ int red[4];
    const int PP = T + 4;
    const int i = threadIdx.x, bh = blockIdx.x, b = bh / H, h = bh % H, linha0 = b * T, ld = 3 * D, ldb = ld / blk;
    const size_t lin = (size_t)(linha0 + i);
    const int emg = max_cta((int)goE[lin * (D / blk) + (h * HD) / blk], red, i);
    const int emq = max_cta((int)qE[lin * ldb + (h * HD) / blk], red, i);
    const int emk = max_cta((int)qE[lin * ldb + (D + h * HD) / blk], red, i);
    const int emv = max_cta((int)qE[lin * ldb + (2 * D + h * HD) / blk], red, i);
    int g[HD], v[HD], q[HD], t[HD];
    linha_alinhada<HD>(gom, goE, lin, D, blk, h * HD, emg, GA, g);
    linha_alinhada<HD>(qm, qE, lin, ld, blk, h * HD, emq, GA, q);
    linha_alinhada<HD>(qm, qE, lin, ld, blk, D + h * HD, emk, GA, t);
    linha_alinhada<HD>(qm, qE, lin, ld, blk, 2 * D + h * HD, emv, GA, v);
    guarda<HD>(g_s + i * HD, g);
    guarda<HD>(q_s + i * HD, q);
    guarda<HD>(k_s + i * HD, t);
    guarda<HD>(v_s + i * HD, v);
    {   // P of this head, key-major rows of T bytes -> shared memory rows of T + 4 bytes (a word per access)
        const uint32_t* Pg = reinterpret_cast<const uint32_t*>(P + (size_t)bh * T * T);
        for (int k = i; k < T * T / 4; k += T) {
            const int j = (k * 4) / T, c = (k * 4) % T;
            *reinterpret_cast<uint32_t*>(P_s + j * PP + c) = Pg[k];
        }
    }
    __syncthreads();
    // shift of gP (to 15 bits): from its exact maximum over j <= i, or from the bounds of the upper-bound variant (ops.py:231-235)
    int sh;
    if (limite) {
        int mg = 0, s1 = 0;
#pragma unroll
        for (int k = 0; k < HD; k++) { mg = max(mg, g[k] < 0 ? -g[k] : g[k]); s1 += v[k] < 0 ? -v[k] : v[k]; }
        sh = max(bitlen(max_cta(mg, red, i) * max_cta(s1, red, i)) - 15, 0);
    } else {
        int mgp = 0;
        for (int j = 0; j <= i; j++) {
            const int gp = ponto<HD>(g, v_s + j * HD);
            mgp = max(mgp, gp < 0 ? -gp : gp);
        }
        sh = max(bitlen(max_cta(mgp, red, i)) - 15, 0);
    }
    // s_lin of this row, then the maxima that give the shift of dS (to 12 bits) (ops.py:236-244)
    int s = 0, mgq = 0;
    for (int j = 0; j <= i; j++) {
        const int gp = rnd_d(ponto<HD>(g, v_s + j * HD), sh);
        s += (int)P_s[j * PP + i] * gp;
        mgq = max(mgq, gp < 0 ? -gp : gp);
    }
    const int sl = rnd_d(s, 8);
    sl_s[i] = sl;
    int mds = 0, mp = 0;
    for (int j = 0; j <= i; j++) {
        const int p = P_s[j * PP + i], ds = p * (rnd_d(ponto<HD>(g, v_s + j * HD), sh) - sl);
        mds = max(mds, ds < 0 ? -ds : ds);
        mp = max(mp, p);
    }
    int sh2;
    if (limite) sh2 = max(bitlen(max_cta(mp, red, i) * (max_cta(mgq, red, i) + max_cta(sl < 0 ? -sl : sl, red, i))) - 12, 0);
    else sh2 = max(bitlen(max_cta(mds, red, i)) - 12, 0);
    const int eds = (emg - GA) + (emv - GA) + sh - 9 + sh2;
    // gq of this row
    int o[HD];
#pragma unroll
    for (int k = 0; k < HD; k++) o[k] = 0;
    for (int j = 0; j <= i; j++) {
        const int ds = rnd_d((int)P_s[j * PP + i] * (rnd_d(ponto<HD>(g, v_s + j * HD), sh) - sl), sh2);
        const int* kj = k_s + j * HD;
#pragma unroll
        for (int k4 = 0; k4 < HD / 4; k4++) {
            const int4 w = reinterpret_cast<const int4*>(kj)[k4];
            o[4 * k4] += ds * w.x; o[4 * k4 + 1] += ds * w.y; o[4 * k4 + 2] += ds * w.z; o[4 * k4 + 3] += ds * w.w;
        }
    }
    grava_cru<HD>(Gacc, Ge, (size_t)lin * 3 * D + h * HD, o, eds + (emk - GA));
    __syncthreads();                                               // sl_s complete
    // thread = key j: gk[j] = sum_{i >= j} dS'[i][j] q[i], gv[j] = sum_{i >= j} P[i][j] dO[i]
    const int j = i;
    int gk[HD], gv[HD];
#pragma unroll
    for (int k = 0; k < HD; k++) gk[k] = gv[k] = 0;
    for (int ii = j; ii < T; ii++) {
        const int p = P_s[j * PP + ii];
        const int* gi = g_s + ii * HD;
        const int* qi = q_s + ii * HD;
        int gp = 0;
#pragma unroll
        for (int k4 = 0; k4 < HD / 4; k4++) {
            const int4 w = reinterpret_cast<const int4*>(gi)[k4];
            gp += w.x * v[4 * k4] + w.y * v[4 * k4 + 1] + w.z * v[4 * k4 + 2] + w.w * v[4 * k4 + 3];
            gv[4 * k4] += p * w.x; gv[4 * k4 + 1] += p * w.y; gv[4 * k4 + 2] += p * w.z; gv[4 * k4 + 3] += p * w.w;
        }
        const int ds = rnd_d(p * (rnd_d(gp, sh) - sl_s[ii]), sh2);
#pragma unroll
        for (int k4 = 0; k4 < HD / 4; k4++) {
            const int4 w = reinterpret_cast<const int4*>(qi)[k4];
            gk[4 * k4] += ds * w.x; gk[4 * k4 + 1] += ds * w.y; gk[4 * k4 + 2] += ds * w.z; gk[4 * k4 + 3] += ds * w.w;
        }
    }
    grava_cru<HD>(Gacc, Ge, (size_t)lin * 3 * D + D + h * HD, gk, eds + (emq - GA));
    grava_cru<HD>(Gacc, Ge, (size_t)lin * 3 * D + 2 * D + h * HD, gv, (emg - GA) - 8);
}
inline size_t smem_back_peq(int HD, int T) { return (size_t)4 * T * HD * 4 + (size_t)T * 4 + (size_t)T * (T + 4); }

}  // namespace atp

static bool atp_serve(int blk, int T, int H, int D) {
    const int hd = H > 0 ? D / H : 0;
    return H > 0 && D == H * hd && (hd == 4 || hd == 16) && T % 32 == 0 && T <= atp::TMAX && D % blk == 0 && blk % hd == 0;
}
static int atp_lg2(int hd) { return hd == 4 ? 2 : 4; }

static int atencao_frente_peq(int blk, const int8_t* qm, const int8_t* qE, int* Oacc, int16_t* Oe, uint8_t* P, int Bt, int T, int H, int D, int GA,
                              int kid, cudaStream_t st) {
    const int hd = D / H;
    if (hd == 4) atp::k_atencao_peq<4><<<Bt * H, T, 0, st>>>(qm, qE, Oacc, Oe, P, T, H, D, GA, blk, atp_lg2(hd), kid);
    else atp::k_atencao_peq<16><<<Bt * H, T, 0, st>>>(qm, qE, Oacc, Oe, P, T, H, D, GA, blk, atp_lg2(hd), kid);
    return (int)cudaGetLastError();
}
static int atencao_tras_peq(int blk, const int8_t* gom, const int8_t* goE, const int8_t* qm, const int8_t* qE, const uint8_t* P, int* Gacc, int16_t* Ge,
                            int Bt, int T, int H, int D, int GA, int limite, int kid, cudaStream_t st) {
    const int hd = D / H;
    const size_t sm = atp::smem_back_peq(hd, T);
    cudaError_t c;
    if (hd == 4) {
        if ((c = at_smem(atp::k_atencao_back_peq<4>, sm)) != cudaSuccess) return (int)c;
        atp::k_atencao_back_peq<4><<<Bt * H, T, sm, st>>>(gom, goE, qm, qE, P, Gacc, Ge, T, H, D, GA, blk, limite, kid);
    } else {
        if ((c = at_smem(atp::k_atencao_back_peq<16>, sm)) != cudaSuccess) return (int)c;
        atp::k_atencao_back_peq<16><<<Bt * H, T, sm, st>>>(gom, goE, qm, qE, P, Gacc, Ge, T, H, D, GA, blk, limite, kid);
    }
    return (int)cudaGetLastError();
}

}  // namespace jt
