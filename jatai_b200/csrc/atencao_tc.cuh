// Integer causal attention with ALiBi on the tensor cores (tcgen05.mma kind::i8, accumulators in tensor memory), head dimension 64.
//
// Same specification and layouts as atencao.cuh (jatai_cuda/ops.py:186-258 generalised; jatai_cuda/jatai_cuda.cu:822-1006).  What
// changes is where the six contractions run.  Every one of them - q.k^T, P.V, dO.v^T, dS'.k, dS'^T.q, P^T.dO - is an exact integer
// sum followed by ONE rounding, so (unlike the block GEMM) a whole contraction can accumulate in tensor memory.  The aligned
// operands have 12 bits (|m << 4| <= 2032) and dS' has 13; kind::i8 takes 8, so each value is split into two signed digits,
//     v = 128 hi + lo,   lo in [-64, 63],   hi in [-32, 32],
// and a product of two split operands is three accumulators: hi.hi, hi.lo + lo.hi, lo.lo, recombined with shifts after the drain
// (all sums stay far below 2^31; the final int32 wraps exactly like the specification's int64 -> int32 truncation).  P is uint8
// and enters as it is (kind::i8 takes u8 x s8).
//
// A preparation kernel aligns q, k, v (and dO) of every head to the head's maximum exponent once, splits them and writes the
// digits to a workspace in the two layouts the MMAs need (both K-major):
//     row layout     [BH*T][128]   token row = [hi digits of the 64 columns | lo digits]     (operand whose K is the head dimension)
//     transposed     [BH*128][T]   row = one digit of one column, over the tokens            (operand whose K is the token axis)
// The attention kernels fetch their tiles from there by TMA (128-byte swizzle) and never touch q, k, v again.
//
// Orientation of every score-like product: tensor-memory lane = key j (M = 128 keys of a chunk), column = query i (N = 32 queries of
// the CTA's row tile); a thread of the drain owns one key and 16 queries.  Stored P is key-major, so that thread reads or writes 16
// contiguous bytes of P.  Products whose output is [token, 64] are computed transposed: lane = digit row of the 64 columns
// (hi rows 0..63, lo rows 64..127), column = token, and recombined through shared memory.
//
// Every mbarrier wait is bounded (sentinel 7, abort flag, normal exit with tensor memory freed), as in the block GEMM.
#pragma once
#include "comum.cuh"
#include "gemm_tc.cuh"
#include "atencao.cuh"

namespace jt {
namespace atc {

using namespace tc;

constexpr int HD = 64, NI = 32, TJ = 128, NJ = 64;
constexpr uint32_t idesc(int n, bool b_sem_sinal) {       // kind::i8, D = s32, A = s8, B = s8 or u8, both K-major, M = 128
    return (2u << 4) | (1u << 7) | ((b_sem_sinal ? 0u : 1u) << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
}
constexpr uint32_t ID_S = idesc(NI, false), ID_PU = idesc(NI, true), ID_C = idesc(NJ, false), ID_CU = idesc(NJ, true);
constexpr uint32_t TILE_A = 128 * 128, TILE_NI = NI * 128, TILE_NJ = NJ * 128;

__device__ __forceinline__ void digitos(int v, int& hi, int& lo) {
    hi = (v + 64) >> 7;
    lo = v - (hi << 7);
}
// byte offset of (row, byte) inside a K-major tile of 128-byte rows with the 128-byte swizzle (8-row groups of 1024 bytes)
__device__ __forceinline__ uint32_t sw128(int linha, int byte) {
    return (uint32_t)((linha >> 3) * 1024 + (linha & 7) * 128 + ((((byte >> 4) ^ (linha & 7)) << 4) | (byte & 15)));
}
__device__ __forceinline__ void fence_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// 16 columns of this thread's lane from three accumulators 32 columns apart (hi.hi, cross, lo.lo)
__device__ __forceinline__ void tmem_le16x3(uint32_t t, uint32_t (&a)[16], uint32_t (&b)[16], uint32_t (&c)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%48];\n"
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%49];\n"
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%32,%33,%34,%35,%36,%37,%38,%39,%40,%41,%42,%43,%44,%45,%46,%47}, [%50];\n"
        "tcgen05.wait::ld.sync.aligned;\n"
        : JT_O16(a, 0), JT_O16(b, 0), JT_O16(c, 0)
        : "r"(t), "r"(t + 32), "r"(t + 64)
        : "memory");
}
__device__ __forceinline__ void tmem_le16(uint32_t t, uint32_t (&a)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];\n"
        "tcgen05.wait::ld.sync.aligned;\n"
        : JT_O16(a, 0)
        : "r"(t)
        : "memory");
}
__device__ __forceinline__ void tmem_aloca(uint32_t* slot, int colunas) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(slot)), "r"(colunas) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_libera(uint32_t tmem, int colunas) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(colunas) : "memory");
}
// the eight MMAs of one score-like product: A = 128 rows of [hi | lo], B = N rows of [hi | lo] -> hi.hi at tm, cross at tm + 32, lo.lo at tm + 64
__device__ __forceinline__ void mma_digitos(uint32_t tm, uint64_t da, uint64_t db, uint32_t id) {
    tc_mma_i8(tm, da, db, id, 0);
    tc_mma_i8(tm, da + 2, db + 2, id, 1);
    tc_mma_i8(tm + 64, da + 4, db + 4, id, 0);
    tc_mma_i8(tm + 64, da + 6, db + 6, id, 1);
    tc_mma_i8(tm + 32, da, db + 4, id, 0);
    tc_mma_i8(tm + 32, da + 2, db + 6, id, 1);
    tc_mma_i8(tm + 32, da + 4, db, id, 1);
    tc_mma_i8(tm + 32, da + 6, db + 2, id, 1);
}
__device__ __forceinline__ int junta3(uint32_t hh, uint32_t cr, uint32_t ll) { return (int)((hh << 14) + (cr << 7) + ll); }

// A kernel whose bounded wait expired has recorded sentinel 7: every CTA that starts afterwards leaves at once instead of waiting
// out its own limit (all threads of the CTA take the same decision).
__device__ __forceinline__ bool ja_parou(int tid) {
    __shared__ int parou;
    if (tid == 0) parou = *reinterpret_cast<volatile int*>(&g_erro.n) != 0 && *reinterpret_cast<volatile int*>(&g_erro.codigo) == E_TEMPO;
    __syncthreads();
    return parou != 0;
}

// -------------------------------------------------------------------------------------------------- preparation
// z = 0 q, 1 k, 2 v (columns of QKV), 3 dO.  Per tensor: destination in row layout and / or transposed layout (nullptr = not needed).
struct ArgsPrep {
    const int8_t* qm; const int8_t* qE; const int8_t* gm; const int8_t* gE;
    int8_t* lin[4]; int8_t* tra[4];
    int* em;                    // [BH][4] head-maximum exponents, indexed by z
    int T, H, D, GA, blk;
};

// grid (ceil(T / 128), BH, 4), 256 threads: 128 tokens of one head of one tensor
__global__ void __launch_bounds__(256) k_at_prep(const ArgsPrep A) {
    __shared__ int red[8];
    __shared__ __align__(16) uint8_t tr[128 * 144];
    const int tid = threadIdx.x, z = blockIdx.z, bh = blockIdx.y, b = bh / A.H, h = bh % A.H, t0 = blockIdx.x * 128;
    int8_t* dl = z == 0 ? A.lin[0] : z == 1 ? A.lin[1] : z == 2 ? A.lin[2] : A.lin[3];
    int8_t* dt = z == 0 ? A.tra[0] : z == 1 ? A.tra[1] : z == 2 ? A.tra[2] : A.tra[3];
    if (!dl && !dt) return;
    const int T = A.T, D = A.D, blk = A.blk, linha0 = b * T;
    const int8_t* m = z == 3 ? A.gm : A.qm;
    const int8_t* E = z == 3 ? A.gE : A.qE;
    const int ld = z == 3 ? D : 3 * D, col0 = z == 3 ? h * HD : z * D + h * HD, ldb = ld / blk;
    const int em = at::max_cabeca<HD>(E, ldb, blk, linha0, T, col0, red, tid);
    if (blockIdx.x == 0 && tid == 0) A.em[bh * 4 + z] = em;
    const int r = tid >> 1, meio = tid & 1, t = t0 + r;
    if (t < T) {
        const size_t lin = (size_t)(linha0 + t);
#pragma unroll
        for (int parte = 0; parte < 2; parte++) {
            const int c = meio * 32 + parte * 16;
            int v[16], hi[16], lo[16];
            le16(m + lin * ld + col0 + c, v);
            const int s = em - (int)E[lin * ldb + (col0 + c) / blk];
#pragma unroll
            for (int k = 0; k < 16; k++) digitos(rnd_d(v[k] << A.GA, s), hi[k], lo[k]);
            if (dl) {
                int8_t* p = dl + ((size_t)bh * T + t) * 128 + c;
                grava16(p, hi);
                grava16(p + 64, lo);
            }
            if (dt) {
#pragma unroll
                for (int k = 0; k < 16; k++) {
                    tr[(c + k) * 144 + r] = (uint8_t)hi[k];
                    tr[(64 + c + k) * 144 + r] = (uint8_t)lo[k];
                }
            }
        }
    }
    if (dt) {
        __syncthreads();
        const int dd = tid >> 1;
#pragma unroll
        for (int q = 0; q < 4; q++) {
            const int off = meio * 64 + q * 16;
            if (t0 + off < T)
                *reinterpret_cast<uint4*>(dt + ((size_t)bh * 128 + dd) * T + t0 + off) = *reinterpret_cast<const uint4*>(tr + dd * 144 + off);
        }
    }
}

// shared-memory carve-up helpers: every operand tile starts on a 1024-byte boundary
struct Barras {
    uint32_t base;
    __device__ uint32_t operator[](int i) const { return base + 8 * i; }
};

// -------------------------------------------------------------------------------------------------- forward
// ops.py:198-219.  grid (T / 32, BH), 256 threads.  Shared: 2 operand stages (K chunks, then V^T chunks; the byte copy of P for
// the store sits on top of them in between), the query tile, P in MMA layout, the scores u[32][T+4] (int32).
// Tensor memory: two score buffers of 3 x 32 columns, one output accumulator of 32 columns (256 allocated).
__global__ void __launch_bounds__(256) k_atencao_tc(const __grid_constant__ CUtensorMap mQ, const __grid_constant__ CUtensorMap mK,
                                                    const __grid_constant__ CUtensorMap mVt, const int* __restrict__ em, int* __restrict__ Oacc,
                                                    int16_t* __restrict__ Oe, uint8_t* __restrict__ P, int T, int H, int D, int GA, int kid) {
    extern __shared__ unsigned char bruto[];
    unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)bruto + 1023) & ~(uintptr_t)1023);
    const uint32_t sbase = smem_u32(smem);
    const int nchT = (T + TJ - 1) / TJ, TP = T + 4;
    const uint32_t OFF_Q = 2 * TILE_A, OFF_PB = OFF_Q + TILE_NI, OFF_U = OFF_PB + nchT * TILE_NI, OFF_BAR = OFF_U + NI * TP * 4;
    uint8_t* pT = smem;                                            // [T][32] bytes, over the operand stages
    uint8_t* pB = smem + OFF_PB;
    int* u_s = reinterpret_cast<int*>(smem + OFF_U);
    const Barras bar = {sbase + OFF_BAR};                          // 0 q | 1,2 k | 3,4 s | 5,6 v | 7,8 v free | 9 o
    uint32_t* slot = reinterpret_cast<uint32_t*>(smem + OFF_BAR + 96);
    volatile int* aborta = reinterpret_cast<volatile int*>(smem + OFF_BAR + 100);
    const int tid = threadIdx.x, wid = tid >> 5, lane = tid & 31;
    const int ordem = blockIdx.y * gridDim.x + blockIdx.x;         // heaviest (last) row tiles of all heads first
    const int bh = ordem % gridDim.y, b = bh / H, h = bh % H, i0 = (gridDim.x - 1 - ordem / gridDim.y) * NI, linha0 = b * T;
    if (ja_parou(tid)) return;
    if (tid == 0) {
        for (int i = 0; i < 10; i++) mbar_init(bar[i], 1);
        *aborta = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (wid == 0) tmem_aloca(slot, 256);
    tc_fence_antes();
    __syncthreads();
    tc_fence_depois();
    const uint32_t tmem = *slot;
    const int emq = em[bh * 4], emk = em[bh * 4 + 1], emv = em[bh * 4 + 2];
    const int s_u = -((emq - GA) + (emk - GA) - 3 + 8), incl = at::incl_alibi(h);
    const int nproc = i0 + NI, nch = (nproc + TJ - 1) / TJ;
    const uint32_t sA[2] = {sbase, sbase + TILE_A}, sQ = sbase + OFF_Q, sPB = sbase + OFF_PB;

    if (tid == 0) {
        mbar_expect_tx(bar[0], TILE_NI);
        tma_2d(sQ, &mQ, 0, bh * T + i0, bar[0]);
        for (int c = 0; c < 2 && c < nch; c++) {
            mbar_expect_tx(bar[1 + c], TILE_A);
            tma_2d(sA[c], &mK, 0, bh * T + c * TJ, bar[1 + c]);
        }
    }
    auto emite = [&](int c) -> bool {                              // one thread: the score MMAs of key chunk c
        if (c == 0 && !espera(bar[0], 0, aborta, kid, 20)) return false;
        if (!espera(bar[1 + (c & 1)], (c >> 1) & 1, aborta, kid, 21)) return false;
        tc_fence_depois();
        mma_digitos(tmem + (c & 1) * 96, desc_sw128(sA[c & 1]), desc_sw128(sQ), ID_S);
        tc_commit(bar[3 + (c & 1)]);
        return true;
    };
    bool ok = true;
    if (tid == 0) ok = emite(0);
    for (int c = 0; c < nch; c++) {
        if (tid == 0 && ok && c + 1 < nch) ok = emite(c + 1);
        __syncwarp();
        ok = __all_sync(FULL, ok && espera(bar[3 + (c & 1)], (c >> 1) & 1, aborta, kid, 22));
        tc_fence_depois();
        if (tid == 0 && ok && c + 2 < nch) {                       // chunk c's MMAs are done: its stage takes chunk c + 2
            mbar_expect_tx(bar[1 + (c & 1)], TILE_A);
            tma_2d(sA[c & 1], &mK, 0, bh * T + (c + 2) * TJ, bar[1 + (c & 1)]);
        }
        if (ok) {
            const int jl = 32 * (wid & 3) + lane, g = wid >> 2, j = c * TJ + jl;
            uint32_t hh[16], cr[16], ll[16];
            tmem_le16x3(tmem + ((uint32_t)(32 * (wid & 3)) << 16) + (c & 1) * 96 + 16 * g, hh, cr, ll);
            if (j < nproc) {
#pragma unroll
                for (int k = 0; k < 16; k++) {
                    const int i = i0 + 16 * g + k;
                    int u = U_MIN;
                    if (j <= i) u = rnd(junta3(hh[k], cr[k], ll[k]), s_u, kid, (long long)(linha0 + i) * D + h * HD) - ((i - j) << incl);
                    u_s[(16 * g + k) * TP + j] = u;
                }
            }
        }
        tc_fence_antes();
        __syncthreads();
    }
    // softmax of the 4 rows of this warp (ops.py:210-217); P goes to pB (MMA operand layout) and to pT (the stored layout)
    const int npad = nch * TJ;
#pragma unroll
    for (int r = 0; r < 4; r++) {
        const int row = 4 * wid + r, i = i0 + row;
        int* ur = u_s + row * TP;
        int m = U_MIN;
        for (int j = lane; j < nproc; j += 32) m = max(m, ur[j]);
        m = warp_max(m);
        int soma = 0;
        for (int j = lane; j < nproc; j += 32) {
            const int ex = j <= i ? exp_dif(m, ur[j]) >> 3 : 0;
            ur[j] = ex;
            soma += ex;
        }
        soma = warp_sum(soma);
        if (soma <= 0) { if (lane == 0) reporta(E_DIV, kid, (long long)(linha0 + i) * D + h * HD, soma, 0); soma = 1; }
        const int inv = (1 << 28) / soma;
        for (int j = lane; j < npad; j += 32) {
            int p = 0;
            if (j < nproc) {
                p = min((ur[j] * inv + (1 << 19)) >> 20, 255);
                pT[j * NI + row] = (uint8_t)p;
            }
            pB[(j >> 7) * TILE_NI + sw128(row, j & 127)] = (uint8_t)p;
        }
    }
    fence_async();                                                 // pB is read by the tensor core (async proxy)
    __syncthreads();
    for (int k = tid; k < T * 2; k += 256) {                       // stored P: for every key the 32 query rows of this tile are contiguous
        const int j = k >> 1, hf = k & 1;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (j < nproc) v = *reinterpret_cast<const uint4*>(pT + j * NI + hf * 16);
        *reinterpret_cast<uint4*>(P + ((size_t)bh * T + j) * T + i0 + hf * 16) = v;
    }
    fence_async();
    __syncthreads();                                               // pT is dead: the stages take the V^T chunks
    // O^T[digit row][query] = sum over keys of V^T . P^T, accumulated over all chunks in tensor memory
    if (tid == 0 && ok) {
        for (int c = 0; c < 2 && c < nch; c++) {
            mbar_expect_tx(bar[5 + c], TILE_A);
            tma_2d(sA[c], &mVt, c * TJ, bh * 128, bar[5 + c]);
        }
        for (int c = 0; c < nch && ok; c++) {
            ok = espera(bar[5 + (c & 1)], (c >> 1) & 1, aborta, kid, 23);
            if (!ok) break;
            tc_fence_depois();
            const uint64_t da = desc_sw128(sA[c & 1]), db = desc_sw128(sPB + c * TILE_NI);
#pragma unroll
            for (int q = 0; q < 4; q++) tc_mma_i8(tmem + 192, da + 2 * q, db + 2 * q, ID_PU, (c | q) != 0);
            tc_commit(bar[7 + (c & 1)]);
            if (c >= 1 && c + 1 < nch) {                           // chunk c - 1's MMAs done: its stage takes chunk c + 1
                ok = espera(bar[7 + ((c - 1) & 1)], ((c - 1) >> 1) & 1, aborta, kid, 24);
                if (!ok) break;
                mbar_expect_tx(bar[5 + ((c + 1) & 1)], TILE_A);
                tma_2d(sA[(c + 1) & 1], &mVt, (c + 1) * TJ, bh * 128, bar[5 + ((c + 1) & 1)]);
            }
        }
        tc_commit(bar[9]);
    }
    __syncwarp();
    ok = __all_sync(FULL, espera(bar[9], 0, aborta, kid, 25));
    tc_fence_depois();
    int* o_s = u_s;                                                // [128 digit rows][33]
    if (ok) {
        uint32_t d[16];
        const int dd = 32 * (wid & 3) + lane, g = wid >> 2;
        tmem_le16(tmem + ((uint32_t)(32 * (wid & 3)) << 16) + 192 + 16 * g, d);
#pragma unroll
        for (int k = 0; k < 16; k++) o_s[dd * 33 + 16 * g + k] = (int)d[k];
    }
    tc_fence_antes();
    __syncthreads();
    {
        const int i = tid >> 3, d0 = (tid & 7) * 8;
        const int eo = (emv - GA) - 8;
        const uint32_t e2 = (uint32_t)(eo & 0xffff) | ((uint32_t)eo << 16);
        int o[8];
#pragma unroll
        for (int k = 0; k < 8; k++) o[k] = (int)(((uint32_t)o_s[(d0 + k) * 33 + i] << 7) + (uint32_t)o_s[(64 + d0 + k) * 33 + i]);
        const size_t p = (size_t)(linha0 + i0 + i) * D + h * HD + d0;
        *reinterpret_cast<int4*>(Oacc + p) = make_int4(o[0], o[1], o[2], o[3]);
        *reinterpret_cast<int4*>(Oacc + p + 4) = make_int4(o[4], o[5], o[6], o[7]);
        *reinterpret_cast<uint4*>(Oe + p) = make_uint4(e2, e2, e2, e2);
    }
    if (wid == 0) {
        tc_fence_depois();
        tmem_libera(tmem, 256);
    }
}
inline size_t smem_frente_tc(int T) { return 1024 + 2 * TILE_A + TILE_NI + (size_t)((T + TJ - 1) / TJ) * TILE_NI + (size_t)NI * (T + 4) * 4 + 128; }

// -------------------------------------------------------------------------------------------------- backward, row tiles
struct ArgsTrasTC {
    const uint8_t* P; int* Gacc; int16_t* Ge; int* est; int* sl; const int* em;      // em: [BH][4] = q, k, v, dO
    int8_t* DSh; int8_t* DSl;                                                         // [BH*T][T] digits of dS', key-major (transposed)
    int T, H, D, GA, limite, kid;
};

// FASE 1: max |gP| over j <= i.   FASE 2: s_lin and the maxima of dS (two sweeps over the keys).   FASE 3: dS' (digits to the
// workspace, key-major, for the key-tile kernel) and gq = dS' . k.     grid (T / 32, BH), 256 threads.
// Every sweep recomputes gP = dO . v^T on the tensor core; nothing T x T is kept in shared memory.
// Tensor memory: two score buffers (3 x 32 columns each) + in phase 3 two output accumulators of 32 columns (256 allocated).
template <int FASE>
__global__ void __launch_bounds__(256) k_ab_linhas_tc(const __grid_constant__ CUtensorMap mV, const __grid_constant__ CUtensorMap mG,
                                                      const __grid_constant__ CUtensorMap mKt, const ArgsTrasTC A) {
    extern __shared__ unsigned char bruto[];
    unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)bruto + 1023) & ~(uintptr_t)1023);
    const uint32_t sbase = smem_u32(smem);
    // stages: V chunks [2] | dO tile | (phase 3) K^T chunks [2] | dS' digit tiles [2][hi, lo]
    constexpr uint32_t OFF_G = 2 * TILE_A, OFF_KT = OFF_G + TILE_NI, OFF_DS = OFF_KT + (FASE == 3 ? 2 * TILE_A : 0);
    constexpr uint32_t OFF_BAR = OFF_DS + (FASE == 3 ? 4 * TILE_NI : 0);
    const Barras bar = {sbase + OFF_BAR};                          // 0 dO | 1,2 v | 3,4 s | 5,6 kt | 7,8 gq done | 9 o
    uint32_t* slot = reinterpret_cast<uint32_t*>(smem + OFF_BAR + 96);
    volatile int* aborta = reinterpret_cast<volatile int*>(smem + OFF_BAR + 100);
    int* sl_s = reinterpret_cast<int*>(smem + OFF_BAR + 128);      // [32]
    int* s_acc = sl_s + 32;                                        // [32]
    __shared__ int red[8];
    const int T = A.T, H = A.H, D = A.D, GA = A.GA, kid = A.kid;
    const int tid = threadIdx.x, wid = tid >> 5, lane = tid & 31;
    const int ordem = blockIdx.y * gridDim.x + blockIdx.x;
    const int bh = ordem % gridDim.y, b = bh / H, h = bh % H, i0 = (gridDim.x - 1 - ordem / gridDim.y) * NI, linha0 = b * T;
    int* est = A.est + bh * at::N_EST;
    if (ja_parou(tid)) return;
    if (tid == 0) {
        for (int i = 0; i < 10; i++) mbar_init(bar[i], 1);
        *aborta = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (tid < 32) { s_acc[tid] = 0; sl_s[tid] = FASE == 3 ? A.sl[(size_t)bh * T + i0 + tid] : 0; }
    if (wid == 0) tmem_aloca(slot, 256);
    tc_fence_antes();
    __syncthreads();
    tc_fence_depois();
    const uint32_t tmem = *slot;
    const int emk = A.em[bh * 4 + 1], emv = A.em[bh * 4 + 2], emg = A.em[bh * 4 + 3];
    const int nproc = i0 + NI, nch = (nproc + TJ - 1) / TJ;
    const int nvoltas = FASE == 2 ? 2 * nch : nch;                 // phase 2 sweeps the keys twice
    const int sh = FASE == 1 ? 0 : at::desl1(est, A.limite);
    const int sh2 = FASE == 3 ? at::desl2(est, A.limite) : 0;
    const int nzero = min((nproc + NJ - 1) / NJ * NJ, T);          // phase 3 writes explicit zeros of dS' up to the key tile's end
    const uint32_t sA[2] = {sbase, sbase + TILE_A}, sG = sbase + OFF_G, sKt[2] = {sbase + OFF_KT, sbase + OFF_KT + TILE_A};
    uint8_t* ds_b = smem + OFF_DS;                                 // [2 stages][hi | lo][32 x 128]

    if (tid == 0) {
        mbar_expect_tx(bar[0], TILE_NI);
        tma_2d(sG, &mG, 0, bh * T + i0, bar[0]);
        for (int c = 0; c < 2 && c < nvoltas; c++) {
            mbar_expect_tx(bar[1 + c], TILE_A);
            tma_2d(sA[c], &mV, 0, bh * T + (c % nch) * TJ, bar[1 + c]);
        }
    }
    auto emite = [&](int cc) -> bool {
        if (cc == 0 && !espera(bar[0], 0, aborta, kid, 30)) return false;
        if (!espera(bar[1 + (cc & 1)], (cc >> 1) & 1, aborta, kid, 31)) return false;
        tc_fence_depois();
        mma_digitos(tmem + (cc & 1) * 96, desc_sw128(sA[cc & 1]), desc_sw128(sG), ID_S);
        tc_commit(bar[3 + (cc & 1)]);
        return true;
    };
    int mgp = 0, mds = 0, mp = 0;
    int s_part[16];
#pragma unroll
    for (int k = 0; k < 16; k++) s_part[k] = 0;
    bool ok = true;
    if (tid == 0) ok = emite(0);
    for (int cc = 0; cc < nvoltas; cc++) {
        const int c = cc % nch, st = cc & 1;
        if (tid == 0 && ok && cc + 1 < nvoltas) ok = emite(cc + 1);
        __syncwarp();
        ok = __all_sync(FULL, ok && espera(bar[3 + st], (cc >> 1) & 1, aborta, kid, 32));
        tc_fence_depois();
        if (tid == 0 && ok && cc + 2 < nvoltas) {
            mbar_expect_tx(bar[1 + st], TILE_A);
            tma_2d(sA[st], &mV, 0, bh * T + ((cc + 2) % nch) * TJ, bar[1 + st]);
        }
        if (FASE == 3) {
            // the stage's digit tiles and K^T chunk are free once the output MMAs of two chunks ago are done
            if (cc >= 2) ok = __all_sync(FULL, ok && espera(bar[7 + st], ((cc - 2) >> 1) & 1, aborta, kid, 33));
            if (tid == 0 && ok) {
                mbar_expect_tx(bar[5 + st], TILE_A);
                tma_2d(sKt[st], &mKt, c * TJ, bh * 128, bar[5 + st]);
            }
        }
        if (FASE == 2 && cc == nch) {
            // between the sweeps: s_lin of the 32 rows from the per-thread partial sums
#pragma unroll
            for (int k = 0; k < 16; k++) {
                const int s = warp_sum(s_part[k]);
                if (lane == 0) atomicAdd(&s_acc[16 * (wid >> 2) + k], s);
            }
            __syncthreads();
            if (tid < 32) {
                const int sl = rnd_d(s_acc[tid], 8);
                sl_s[tid] = sl;
                A.sl[(size_t)bh * T + i0 + tid] = sl;
            }
            __syncthreads();
        }
        if (ok) {
            const int jl = 32 * (wid & 3) + lane, g = wid >> 2, j = c * TJ + jl;
            uint32_t hh[16], cr[16], ll[16];
            tmem_le16x3(tmem + ((uint32_t)(32 * (wid & 3)) << 16) + st * 96 + 16 * g, hh, cr, ll);
            uint32_t pw[4] = {0, 0, 0, 0};
            if (FASE != 1 && j < nproc) {
                const uint4 w = *reinterpret_cast<const uint4*>(A.P + ((size_t)bh * T + j) * T + i0 + 16 * g);
                pw[0] = w.x; pw[1] = w.y; pw[2] = w.z; pw[3] = w.w;
            }
            int dh[16], dl[16];
#pragma unroll
            for (int k = 0; k < 16; k++) {
                const int i = i0 + 16 * g + k;
                const bool dentro = j <= i && j < nproc;
                const int gp = dentro ? rnd_d(junta3(hh[k], cr[k], ll[k]), sh) : 0;
                if (FASE == 1 || (FASE == 2 && cc < nch)) mgp = max(mgp, gp < 0 ? -gp : gp);
                if (FASE == 1) continue;
                const int p = (int)((pw[k >> 2] >> (8 * (k & 3))) & 0xff);
                if (FASE == 2) {
                    if (cc < nch) s_part[k] += p * gp;
                    else {
                        const int ds = p * (gp - sl_s[16 * g + k]);
                        mds = max(mds, ds < 0 ? -ds : ds);
                        mp = max(mp, p);
                    }
                } else {
                    const int ds = dentro ? rnd_d(p * (gp - sl_s[16 * g + k]), sh2) : 0;
                    digitos(ds, dh[k], dl[k]);
                    ds_b[(2 * st) * TILE_NI + sw128(16 * g + k, jl)] = (uint8_t)dh[k];
                    ds_b[(2 * st + 1) * TILE_NI + sw128(16 * g + k, jl)] = (uint8_t)dl[k];
                }
            }
            if (FASE == 3 && j < nzero) {
                const size_t o = ((size_t)bh * T + j) * T + i0 + 16 * g;
                grava16(A.DSh + o, dh);
                grava16(A.DSl + o, dl);
            }
        }
        if (FASE == 3) fence_async();
        tc_fence_antes();
        __syncthreads();
        if (FASE == 3 && tid == 0 && ok) {
            // gq^T[digit row of k][query] += K^T chunk . (dS' digits)^T
            ok = espera(bar[5 + st], (cc >> 1) & 1, aborta, kid, 34);
            if (ok) {
                tc_fence_depois();
                const uint64_t da = desc_sw128(sKt[st]), dbh = desc_sw128(sbase + OFF_DS + (2 * st) * TILE_NI), dbl = desc_sw128(sbase + OFF_DS + (2 * st + 1) * TILE_NI);
#pragma unroll
                for (int q = 0; q < 4; q++) {
                    tc_mma_i8(tmem + 192, da + 2 * q, dbh + 2 * q, ID_S, (cc | q) != 0);
                    tc_mma_i8(tmem + 224, da + 2 * q, dbl + 2 * q, ID_S, (cc | q) != 0);
                }
                tc_commit(bar[7 + st]);
                if (cc == nvoltas - 1) tc_commit(bar[9]);
            }
        }
    }
    if (FASE == 1) {
        at::max_cta_atomico(mgp, est + at::S_GP, red, tid);
    } else if (FASE == 2) {
        int msl = 0;
        if (tid < 32) msl = sl_s[tid] < 0 ? -sl_s[tid] : sl_s[tid];
        at::max_cta_atomico(mds, est + at::S_DS, red, tid);
        if (A.limite) {
            at::max_cta_atomico(mp, est + at::S_P, red, tid);
            at::max_cta_atomico(mgp, est + at::S_GPQ, red, tid);
            at::max_cta_atomico(msl, est + at::S_SL, red, tid);
        }
    } else {
        __syncwarp();
        ok = __all_sync(FULL, ok && espera(bar[9], 0, aborta, kid, 35));
        tc_fence_depois();
        int* o_s = reinterpret_cast<int*>(smem);                   // [2][128][33] over the dead operand stages
        if (ok) {
            uint32_t d1[16], d2[16];
            const int dd = 32 * (wid & 3) + lane, g = wid >> 2;
            const uint32_t t = tmem + ((uint32_t)(32 * (wid & 3)) << 16) + 192 + 16 * g;
            tmem_le16(t, d1);
            tmem_le16(t + 32, d2);
#pragma unroll
            for (int k = 0; k < 16; k++) {
                o_s[dd * 33 + 16 * g + k] = (int)d1[k];
                o_s[128 * 33 + dd * 33 + 16 * g + k] = (int)d2[k];
            }
        }
        tc_fence_antes();
        __syncthreads();
        const int i = tid >> 3, d0 = (tid & 7) * 8;
        const int eds = (emg - GA) + (emv - GA) + sh - 9 + sh2, e = eds + (emk - GA);
        const uint32_t e2 = (uint32_t)(e & 0xffff) | ((uint32_t)e << 16);
        int o[8];
#pragma unroll
        for (int k = 0; k < 8; k++) {
            const int d = d0 + k;
            const uint32_t hhv = (uint32_t)o_s[d * 33 + i], crv = (uint32_t)o_s[(64 + d) * 33 + i] + (uint32_t)o_s[128 * 33 + d * 33 + i],
                           llv = (uint32_t)o_s[128 * 33 + (64 + d) * 33 + i];
            o[k] = junta3(hhv, crv, llv);
        }
        const size_t p = (size_t)(linha0 + i0 + i) * 3 * D + h * HD + d0;
        *reinterpret_cast<int4*>(A.Gacc + p) = make_int4(o[0], o[1], o[2], o[3]);
        *reinterpret_cast<int4*>(A.Gacc + p + 4) = make_int4(o[4], o[5], o[6], o[7]);
        *reinterpret_cast<uint4*>(A.Ge + p) = make_uint4(e2, e2, e2, e2);
    }
    tc_fence_antes();
    __syncthreads();
    if (wid == 0) {
        tc_fence_depois();
        tmem_libera(tmem, 256);
    }
}
inline size_t smem_linhas_tc(int fase) { return 1024 + 2 * TILE_A + TILE_NI + (fase == 3 ? 2 * TILE_A + 4 * TILE_NI : 0) + 384; }

// -------------------------------------------------------------------------------------------------- backward, key tiles
// gk[j] = sum_i dS'[i][j] q[i], gv[j] = sum_i P[i][j] dO[i] for the 64 keys of the tile, over the query chunks from the tile's first
// key on (everything before is causally zero).  All five operands come by TMA: q^T and dO^T digit rows (A), the tile's rows of the
// dS' digits and of P (B).  grid (ceil(T / 64), BH), 256 threads; tensor memory: three accumulators of 64 columns (256 allocated).
__global__ void __launch_bounds__(256) k_ab_colunas_tc(const __grid_constant__ CUtensorMap mQt, const __grid_constant__ CUtensorMap mGt,
                                                       const __grid_constant__ CUtensorMap mDh, const __grid_constant__ CUtensorMap mDl,
                                                       const __grid_constant__ CUtensorMap mP, const ArgsTrasTC A) {
    extern __shared__ unsigned char bruto[];
    unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)bruto + 1023) & ~(uintptr_t)1023);
    const uint32_t sbase = smem_u32(smem);
    constexpr uint32_t STAGE = 2 * TILE_A + 3 * TILE_NJ, OFF_BAR = 2 * STAGE;
    const Barras bar = {sbase + OFF_BAR};                          // 0,1 full | 2,3 free | 4 o
    uint32_t* slot = reinterpret_cast<uint32_t*>(smem + OFF_BAR + 64);
    volatile int* aborta = reinterpret_cast<volatile int*>(smem + OFF_BAR + 68);
    const int T = A.T, H = A.H, D = A.D, GA = A.GA, kid = A.kid;
    const int tid = threadIdx.x, wid = tid >> 5, lane = tid & 31;
    const int ordem = blockIdx.y * gridDim.x + blockIdx.x;         // heaviest (first) key tiles of all heads first
    const int bh = ordem % gridDim.y, b = bh / H, h = bh % H, j0 = (ordem / gridDim.y) * NJ, linha0 = b * T;
    const int* est = A.est + bh * at::N_EST;
    if (ja_parou(tid)) return;
    if (tid == 0) {
        for (int i = 0; i < 5; i++) mbar_init(bar[i], 1);
        *aborta = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (wid == 0) tmem_aloca(slot, 256);
    tc_fence_antes();
    __syncthreads();
    tc_fence_depois();
    const uint32_t tmem = *slot;
    const int nq = (T - j0 + TJ - 1) / TJ;
    if (tid == 0) {
        auto carrega = [&](int c) {
            const uint32_t s = sbase + (c & 1) * STAGE, f = bar[c & 1];
            const int ic = j0 + c * TJ;
            mbar_expect_tx(f, STAGE);
            tma_2d(s, &mQt, ic, bh * 128, f);
            tma_2d(s + TILE_A, &mGt, ic, bh * 128, f);
            tma_2d(s + 2 * TILE_A, &mDh, ic, bh * T + j0, f);
            tma_2d(s + 2 * TILE_A + TILE_NJ, &mDl, ic, bh * T + j0, f);
            tma_2d(s + 2 * TILE_A + 2 * TILE_NJ, &mP, ic, bh * T + j0, f);
        };
        for (int c = 0; c < 2 && c < nq; c++) carrega(c);
        bool ok = true;
        for (int c = 0; c < nq && ok; c++) {
            ok = espera(bar[c & 1], (c >> 1) & 1, aborta, kid, 40);
            if (!ok) break;
            tc_fence_depois();
            const uint32_t s = sbase + (c & 1) * STAGE;
            const uint64_t dq = desc_sw128(s), dg = desc_sw128(s + TILE_A), dh = desc_sw128(s + 2 * TILE_A), dl = desc_sw128(s + 2 * TILE_A + TILE_NJ),
                           dp = desc_sw128(s + 2 * TILE_A + 2 * TILE_NJ);
#pragma unroll
            for (int q = 0; q < 4; q++) {
                tc_mma_i8(tmem, dq + 2 * q, dh + 2 * q, ID_C, (c | q) != 0);
                tc_mma_i8(tmem + 64, dq + 2 * q, dl + 2 * q, ID_C, (c | q) != 0);
                tc_mma_i8(tmem + 128, dg + 2 * q, dp + 2 * q, ID_CU, (c | q) != 0);
            }
            tc_commit(bar[2 + (c & 1)]);
            if (c >= 1 && c + 1 < nq) {
                ok = espera(bar[2 + ((c - 1) & 1)], ((c - 1) >> 1) & 1, aborta, kid, 41);
                if (ok) carrega(c + 1);
            }
        }
        tc_commit(bar[4]);
    }
    __syncwarp();
    const bool ok = __all_sync(FULL, espera(bar[4], 0, aborta, kid, 42));
    tc_fence_depois();
    int* o_s = reinterpret_cast<int*>(smem);                       // [3][128][65] over the dead stages
    if (ok) {
        const int dd = 32 * (wid & 3) + lane, g = wid >> 2;        // 32 of the 64 columns per thread
#pragma unroll
        for (int a = 0; a < 3; a++) {
            uint32_t d[32];
            tmem_le32(tmem + ((uint32_t)(32 * (wid & 3)) << 16) + 64 * a + 32 * g, d);
#pragma unroll
            for (int k = 0; k < 32; k++) o_s[(a * 128 + dd) * 65 + 32 * g + k] = (int)d[k];
        }
    }
    tc_fence_antes();
    __syncthreads();
    {
        const int sh = at::desl1(est, A.limite), sh2 = at::desl2(est, A.limite);
        const int emq = A.em[bh * 4], emv = A.em[bh * 4 + 2], emg = A.em[bh * 4 + 3];
        const int ego = emg - GA, eds = ego + (emv - GA) + sh - 9 + sh2, e_k = eds + (emq - GA), e_v = ego - 8;
        const uint32_t k2 = (uint32_t)(e_k & 0xffff) | ((uint32_t)e_k << 16), v2 = (uint32_t)(e_v & 0xffff) | ((uint32_t)e_v << 16);
        for (int t = tid; t < NJ * 8; t += 256) {
            const int jl = t >> 3, d0 = (t & 7) * 8, j = j0 + jl;
            if (j >= T) continue;
            int gk[8], gv[8];
#pragma unroll
            for (int k = 0; k < 8; k++) {
                const int d = d0 + k;
                const uint32_t hhv = (uint32_t)o_s[d * 65 + jl], crv = (uint32_t)o_s[(64 + d) * 65 + jl] + (uint32_t)o_s[(128 + d) * 65 + jl],
                               llv = (uint32_t)o_s[(128 + 64 + d) * 65 + jl];
                gk[k] = junta3(hhv, crv, llv);
                gv[k] = (int)(((uint32_t)o_s[(256 + d) * 65 + jl] << 7) + (uint32_t)o_s[(256 + 64 + d) * 65 + jl]);
            }
            const size_t p = (size_t)(linha0 + j) * 3 * D + D + h * HD + d0;
            *reinterpret_cast<int4*>(A.Gacc + p) = make_int4(gk[0], gk[1], gk[2], gk[3]);
            *reinterpret_cast<int4*>(A.Gacc + p + 4) = make_int4(gk[4], gk[5], gk[6], gk[7]);
            *reinterpret_cast<uint4*>(A.Ge + p) = make_uint4(k2, k2, k2, k2);
            *reinterpret_cast<int4*>(A.Gacc + p + D) = make_int4(gv[0], gv[1], gv[2], gv[3]);
            *reinterpret_cast<int4*>(A.Gacc + p + D + 4) = make_int4(gv[4], gv[5], gv[6], gv[7]);
            *reinterpret_cast<uint4*>(A.Ge + p + D) = make_uint4(v2, v2, v2, v2);
        }
    }
    if (wid == 0) {
        tc_fence_depois();
        tmem_libera(tmem, 256);
    }
}
inline size_t smem_colunas_tc() { return 1024 + 2 * (2 * TILE_A + 3 * TILE_NJ) + 128; }

}  // namespace atc

// -------------------------------------------------------------------------------------------------- host side
static size_t atc_arredonda(size_t x) { return (x + 1023) & ~(size_t)1023; }

// head dimension 64 and at least one full key chunk (the TMA boxes are 128 tokens wide)
static bool atc_serve(int blk, int T, int H, int D) { return D == H * atc::HD && T % 32 == 0 && T >= 128 && T <= 1024 && D % blk == 0 && (blk == 32 || blk == 128); }

// forward: preparation (q, k row layout; v transposed) + the tensor-core kernel
static int atencao_frente_tc(int blk, const int8_t* qm, const int8_t* qE, int* Oacc, int16_t* Oe, uint8_t* P, int Bt, int T, int H, int D, int GA,
                             int kid, cudaStream_t st) {
    const int BH = Bt * H;
    const size_t b_em = atc_arredonda((size_t)BH * 16), b_lin = atc_arredonda((size_t)BH * T * 128);
    unsigned char* ws = nullptr;
    if (int r = at_ws(b_em + 3 * b_lin, st, reinterpret_cast<void**>(&ws))) return r;
    int* em = reinterpret_cast<int*>(ws);
    int8_t *Q2 = reinterpret_cast<int8_t*>(ws + b_em), *K2 = Q2 + b_lin, *Vt2 = K2 + b_lin;
    atc::ArgsPrep Pp = {qm, qE, nullptr, nullptr, {Q2, K2, nullptr, nullptr}, {nullptr, nullptr, Vt2, nullptr}, em, T, H, D, GA, blk};
    atc::k_at_prep<<<dim3((T + 127) / 128, BH, 3), 256, 0, st>>>(Pp);
    CUtensorMap mQ, mK, mVt;
    if (!(faz_mapa(&mQ, Q2, BH * T, 128, atc::NI) && faz_mapa(&mK, K2, BH * T, 128, 128) && faz_mapa(&mVt, Vt2, BH * 128, T, 128)))
        return (int)cudaErrorInvalidValue;
    const size_t sm = atc::smem_frente_tc(T);
    cudaError_t c = at_smem(atc::k_atencao_tc, sm);
    if (c != cudaSuccess) return (int)c;
    atc::k_atencao_tc<<<dim3(T / atc::NI, BH), 256, sm, st>>>(mQ, mK, mVt, em, Oacc, Oe, P, T, H, D, GA, kid);
    return (int)cudaGetLastError();
}

// backward: preparation (v, dO row layout; q, k, dO transposed), the three row-tile phases, the key-tile kernel
static int atencao_tras_tc(int blk, const int8_t* gom, const int8_t* goE, const int8_t* qm, const int8_t* qE, const uint8_t* P, int* Gacc, int16_t* Ge,
                           int Bt, int T, int H, int D, int GA, int limite, int kid, cudaStream_t st) {
    const int BH = Bt * H;
    const size_t b_est = atc_arredonda((size_t)BH * (at::N_EST + T + 4) * sizeof(int)), b_lin = atc_arredonda((size_t)BH * T * 128),
                 b_ds = atc_arredonda((size_t)BH * T * T);
    unsigned char* ws = nullptr;
    if (int r = at_ws(b_est + 5 * b_lin + 2 * b_ds, st, reinterpret_cast<void**>(&ws))) return r;
    int* est = reinterpret_cast<int*>(ws);
    int* sl = est + (size_t)BH * at::N_EST;
    int* em = sl + (size_t)BH * T;
    int8_t *V2 = reinterpret_cast<int8_t*>(ws + b_est), *G2 = V2 + b_lin, *Qt2 = G2 + b_lin, *Kt2 = Qt2 + b_lin, *Gt2 = Kt2 + b_lin;
    int8_t *DSh = Gt2 + b_lin, *DSl = DSh + b_ds;
    cudaError_t c = cudaMemsetAsync(est, 0, (size_t)BH * at::N_EST * sizeof(int), st);
    if (c != cudaSuccess) return (int)c;
    atc::ArgsPrep Pp = {qm, qE, gom, goE, {nullptr, nullptr, V2, G2}, {Qt2, Kt2, nullptr, Gt2}, em, T, H, D, GA, blk};
    atc::k_at_prep<<<dim3((T + 127) / 128, BH, 4), 256, 0, st>>>(Pp);
    CUtensorMap mV, mG, mKt, mQt, mGt, mDh, mDl, mP;
    if (!(faz_mapa(&mV, V2, BH * T, 128, 128) && faz_mapa(&mG, G2, BH * T, 128, atc::NI) && faz_mapa(&mKt, Kt2, BH * 128, T, 128) &&
          faz_mapa(&mQt, Qt2, BH * 128, T, 128) && faz_mapa(&mGt, Gt2, BH * 128, T, 128) && faz_mapa(&mDh, DSh, BH * T, T, atc::NJ) &&
          faz_mapa(&mDl, DSl, BH * T, T, atc::NJ) && faz_mapa(&mP, P, BH * T, T, atc::NJ)))
        return (int)cudaErrorInvalidValue;
    atc::ArgsTrasTC A = {P, Gacc, Ge, est, sl, em, DSh, DSl, T, H, D, GA, limite, kid};
    const dim3 grade(T / atc::NI, BH);
    if (limite) {
        at::ArgsTras L = {gom, goE, qm, qE, P, Gacc, Ge, est, sl, nullptr, T, H, D, GA, blk, limite, kid};
        at::k_lim<atc::HD><<<BH, 256, 0, st>>>(L);
    } else {
        if ((c = at_smem(atc::k_ab_linhas_tc<1>, atc::smem_linhas_tc(1))) != cudaSuccess) return (int)c;
        atc::k_ab_linhas_tc<1><<<grade, 256, atc::smem_linhas_tc(1), st>>>(mV, mG, mKt, A);
    }
    if ((c = at_smem(atc::k_ab_linhas_tc<2>, atc::smem_linhas_tc(2))) != cudaSuccess) return (int)c;
    atc::k_ab_linhas_tc<2><<<grade, 256, atc::smem_linhas_tc(2), st>>>(mV, mG, mKt, A);
    if ((c = at_smem(atc::k_ab_linhas_tc<3>, atc::smem_linhas_tc(3))) != cudaSuccess) return (int)c;
    atc::k_ab_linhas_tc<3><<<grade, 256, atc::smem_linhas_tc(3), st>>>(mV, mG, mKt, A);
    if ((c = at_smem(atc::k_ab_colunas_tc, atc::smem_colunas_tc())) != cudaSuccess) return (int)c;
    atc::k_ab_colunas_tc<<<dim3((T + atc::NJ - 1) / atc::NJ, BH), 256, atc::smem_colunas_tc(), st>>>(mQt, mGt, mDh, mDl, mP, A);
    return (int)cudaGetLastError();
}

}  // namespace jt
