// Output stage shared by the GEMM kernels: raw accumulators of a CTA tile (int32 in shared memory) ->
// block / raw / fused outputs in global memory.
//
// The fused modes are, by definition of the reference, the composition of the separate operations on the
// already quantised GEMM output (jatai_cuda/ops.py:110-119; jatai_cuda/jatai_cuda.cu:201-208 lists the modes):
//   0 block  | 1 raw (int32 + int16 exponent per element, optionally split-K with atomic adds)
//   2 block + residual add  C = soma(X, A.B^T)            | 3 block + ReLU^2: C = h = A.B^T and O2 = relu2(h)
//   4 ReLU^2 backward  C = relu2_back(A.B^T, X) with X = h of the forward.
#pragma once
#include "comum.cuh"

namespace jt {

constexpr int GG = 4;            // guard bits of a K-block partial product (ops.py:104)
constexpr int TN = 128;          // tile width of every GEMM kernel (columns of C per CTA)
constexpr int PITCH = TN + 4;    // row pitch (words) of the staged accumulators: 16-byte aligned rows, conflict-free

struct SaidaGemm {
    int8_t* Cm; int8_t* CE; int* C32; int16_t* Ce;
    const int8_t* Xm; const int8_t* XE; int8_t* Om2; int8_t* OE2;
};

// Called by NTH threads (whole warps, `tid` in [0, NTH)) after the staged tile is visible to all of them.
// Task = 16 consecutive columns of one row.  Within a warp lane l takes row (l % RPW) and chunk (l / RPW) of a
// group of RPW rows (4 rows of a 128-column tile, 8 of a 64-column one), so the 8 lanes of a shared-memory phase
// read different rows (no bank conflict) while the lanes that share a row still write contiguous bytes; the
// lanes of one exponent block sit RPW apart.
//
// Fast path of the block outputs (taken by a whole warp or not at all): when every accumulator of the warp's rows is
// below 2^24 and the column exponents of each block spread over at most 64, the values acc * 2^(RB_j - min RB) are exact
// in fp32 and the fp32 quantiser gives the bits of the integer one.  It needs, from the caller, RBf[j] = 2^(RB_j - min
// of j's block) and RBm[b] = that minimum, RBm[4 + b] = the block's maximum; RBf == nullptr disables it.
template <int BLK, int MODO, int NTH, int TNv = TN>
__device__ __forceinline__ void epilogo_tile(const int* acc_s, const int* RAs, const int* RBs, int linhas, int m0, int n0, int N,
                                             const SaidaGemm& S, bool atomico, bool grava_e, int kid, int tid,
                                             const float* RBf = nullptr, const int* RBm = nullptr) {
    constexpr int GL = BLK / 16;
    constexpr int RPW = 512 / TNv;             // rows a warp handles per iteration: 32 lanes / (TNv / 16) chunks per row
    constexpr int PITCHv = TNv + 4;
    const int lane = tid & 31, wp = tid >> 5;
    const int nW = NTH / 32;
    for (int g4 = wp; g4 < linhas / RPW; g4 += nW) {
        const int r = g4 * RPW + (lane & (RPW - 1)), ch = lane / RPW;
        const int gi = m0 + r, gj = n0 + ch * 16;
        const long long o = (long long)gi * N + gj;
        int v[16];
#pragma unroll
        for (int k = 0; k < 4; k++) {
            const int4 w = *reinterpret_cast<const int4*>(acc_s + r * PITCHv + ch * 16 + 4 * k);
            v[4 * k] = w.x; v[4 * k + 1] = w.y; v[4 * k + 2] = w.z; v[4 * k + 3] = w.w;
        }
        const int ra = RAs[r] - GG;
        if (MODO == 1) {
            if (atomico) {
#pragma unroll
                for (int k = 0; k < 16; k++) if (v[k]) atomicAdd(S.C32 + o + k, v[k]);
            } else {
#pragma unroll
                for (int k = 0; k < 4; k++) reinterpret_cast<int4*>(S.C32 + o)[k] = make_int4(v[4 * k], v[4 * k + 1], v[4 * k + 2], v[4 * k + 3]);
            }
            if (grava_e) {
                uint32_t pk[8];
#pragma unroll
                for (int k = 0; k < 8; k++) {
                    const int e0 = max(ra + RBs[ch * 16 + 2 * k], -30000), e1 = max(ra + RBs[ch * 16 + 2 * k + 1], -30000);
                    pk[k] = (uint32_t)(e0 & 0xffff) | ((uint32_t)e1 << 16);
                }
                reinterpret_cast<uint4*>(S.Ce + o)[0] = make_uint4(pk[0], pk[1], pk[2], pk[3]);
                reinterpret_cast<uint4*>(S.Ce + o)[1] = make_uint4(pk[4], pk[5], pk[6], pk[7]);
            }
            continue;
        }
        const bool lider = (ch % GL) == 0;
        const long long oe = (long long)gi * (N / BLK) + gj / BLK;
        int q[16], E;
        bool rapido = false;
        if (RBf) {
            int amax = 0;
#pragma unroll
            for (int k = 0; k < 16; k++) amax = max(amax, abs(v[k]));
            const int b = ch * 16 / BLK;
            rapido = __all_sync(FULL, amax < (1 << 24) && RBm[4 + b] - RBm[b] <= 64);
            if (rapido) {
                float f[16];
#pragma unroll
                for (int k = 0; k < 4; k++) {
                    const float4 sc = *reinterpret_cast<const float4*>(RBf + ch * 16 + 4 * k);
                    f[4 * k] = (float)v[4 * k] * sc.x; f[4 * k + 1] = (float)v[4 * k + 1] * sc.y;
                    f[4 * k + 2] = (float)v[4 * k + 2] * sc.z; f[4 * k + 3] = (float)v[4 * k + 3] * sc.w;
                }
                uint4 pac;
                E = quant_f32<GL, RPW>(f, ra + RBm[b], pac, kid, o);
                if (MODO == 0 || MODO == 3) {
                    *reinterpret_cast<uint4*>(S.Cm + o) = pac;
                    if (lider) S.CE[oe] = (int8_t)E;
                }
                if (MODO == 0) continue;
                if (MODO == 3) {                   // relu2 of the quantised h (ops.py:134-137): squares <= 16129 are exact in fp32
                    bytes_para_float(pac, f);
#pragma unroll
                    for (int k = 0; k < 16; k++) { const float rr = fmaxf(f[k], 0.f); f[k] = rr * rr; }
                    const int E2 = quant_f32<GL, RPW>(f, 2 * E, pac, kid, o);
                    *reinterpret_cast<uint4*>(S.Om2 + o) = pac;
                    if (lider) S.OE2[oe] = (int8_t)E2;
                    continue;
                }
                if (MODO == 4) {                   // relu2_back (ops.py:139-141): |g h 2| <= 32258
                    float h[16];
                    bytes_para_float(pac, f);
                    bytes_para_float(*reinterpret_cast<const uint4*>(S.Xm + o), h);
#pragma unroll
                    for (int k = 0; k < 16; k++) f[k] = f[k] * fmaxf(h[k], 0.f) * 2.f;
                    const int E2 = quant_f32<GL, RPW>(f, E + (int)S.XE[oe], pac, kid, o);
                    *reinterpret_cast<uint4*>(S.Cm + o) = pac;
                    if (lider) S.CE[oe] = (int8_t)E2;
                    continue;
                }
                desempacota16(pac, q);             // MODO 2 goes on in integers: its sums reach 2^28
            }
        }
        if (!rapido) {
            int e[16];
#pragma unroll
            for (int k = 0; k < 16; k++) e[k] = ra + RBs[ch * 16 + k];
            E = quant_geral<16, GL, RPW>(v, e, q, kid, o);
        }
        if (MODO == 0) {
            grava16(S.Cm + o, q);
            if (lider) S.CE[oe] = (int8_t)E;
        } else if (MODO == 2) {            // soma(X, gemm): ops.py:128-132
            int x[16], z[16];
            le16(S.Xm + o, x);
            const int ex = S.XE[oe], ec = max(ex, E) - 21;
#pragma unroll
            for (int k = 0; k < 16; k++) x[k] = desloca(x[k], ec - ex) + desloca(q[k], ec - E);
            const int E2 = quant_uniforme<16, GL, RPW>(x, ec, z, kid, o);
            grava16(S.Cm + o, z);
            if (lider) S.CE[oe] = (int8_t)E2;
        } else if (MODO == 3) {            // h and relu2(h): ops.py:134-137
            grava16(S.Cm + o, q);
            if (lider) S.CE[oe] = (int8_t)E;
            int a[16], z[16];
#pragma unroll
            for (int k = 0; k < 16; k++) { const int rr = max(q[k], 0); a[k] = rr * rr; }
            const int E2 = quant_uniforme<16, GL, RPW>(a, 2 * E, z, kid, o);
            grava16(S.Om2 + o, z);
            if (lider) S.OE2[oe] = (int8_t)E2;
        } else {                            // relu2_back(gemm, h): ops.py:139-141
            int h[16], z[16];
            le16(S.Xm + o, h);
            const int eh = S.XE[oe];
#pragma unroll
            for (int k = 0; k < 16; k++) h[k] = q[k] * max(h[k], 0) * 2;
            const int E2 = quant_uniforme<16, GL, RPW>(h, E + eh, z, kid, o);
            grava16(S.Cm + o, z);
            if (lider) S.CE[oe] = (int8_t)E2;
        }
    }
}

// row-maximum exponent of `n` int8 values starting at p (16-byte vectors when aligned)
__device__ __forceinline__ int max_expoentes(const int8_t* p, int n) {
    int r = -128;
    int i = 0;
    if ((((uintptr_t)p) & 15) == 0) {
        for (; i + 16 <= n; i += 16) {
            const uint4 w = *reinterpret_cast<const uint4*>(p + i);
            const uint32_t u[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
            for (int k = 0; k < 4; k++) {
                // signed byte maximum of the four lanes of a word
                const unsigned m1 = __vmaxs4(u[k], u[k] >> 16 | u[k] << 16);
                const unsigned m2 = __vmaxs4(m1, m1 >> 8 | m1 << 24);
                r = max(r, (int)(int8_t)(m2 & 0xff));
            }
        }
    }
    for (; i < n; i++) r = max(r, (int)p[i]);
    return r;
}

// R8[i] = max_b E[i, b]: the row-maximum exponents a GEMM aligns to (one thread per row)
__global__ void __launch_bounds__(256) k_max_linha(const int8_t* __restrict__ E, int8_t* __restrict__ R8, int linhas, int nb) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < linhas) R8[i] = (int8_t)max_expoentes(E + (size_t)i * nb, nb);
}

}  // namespace jt
