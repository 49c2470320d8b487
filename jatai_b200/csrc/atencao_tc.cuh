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
// What an MMA costs here: a kind::i8 instruction (M = 128, K = 32) takes ~190 cycles of the SM's tensor pipe whatever its N
// (measured for N = 32 ... 256), so the kernels are built to issue FEW instructions: the B operand is widened instead.  The three
// digit products of a score tile come out of ONE sequence of four instructions (K = 128 bytes of a row [hi | lo]) by stacking
// three arrangements of the query tile as B rows - [qh | 0], [ql | qh], [0 | ql] - so that columns 0..63 of the result are
// hi.hi, 64..127 the cross term and 128..191 lo.lo; likewise the two digits of dS' are stacked as B rows of one tile.
//
// Every mbarrier wait is bounded (sentinel 7, abort flag, normal exit with tensor memory freed), as in the block GEMM.
#pragma once
#include <type_traits>
#include "comum.cuh"
#include "gemm_tc.cuh"
#include "atencao.cuh"

namespace jt {
namespace atc {

using namespace tc;

constexpr int HD = 64, NI = 64, TJ = 128, NJ = 64;
constexpr int NTL = 512;                 // threads of the row-tile kernels: 4 lane quarters x 4 groups of 16 query columns
constexpr int SB = 3 * NI;               // columns of one score buffer in tensor memory: hi.hi | cross | lo.lo
constexpr uint32_t idesc(int n, bool b_sem_sinal) {       // kind::i8, D = s32, A = s8, B = s8 or u8, both K-major, M = 128
    return (2u << 4) | (1u << 7) | ((b_sem_sinal ? 0u : 1u) << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
}
constexpr uint32_t ID_S3 = idesc(SB, false), ID_S2 = idesc(2 * NI, false), ID_PU = idesc(NI, true), ID_C2 = idesc(2 * NJ, false), ID_CU = idesc(NJ, true);
constexpr uint32_t TILE_A = 128 * 128, TILE_NI = NI * 128, TILE_NJ = NJ * 128, TILE_Q3 = 3 * TILE_NI;

__device__ __forceinline__ void digitos(int v, int& hi, int& lo) {
    hi = (v + 64) >> 7;
    lo = v - (hi << 7);
}
// byte offset of (row, byte) inside a K-major tile of 128-byte rows with the 128-byte swizzle (8-row groups of 1024 bytes)
__device__ __forceinline__ uint32_t sw128(int linha, int byte) {
    return (uint32_t)((linha >> 3) * 1024 + (linha & 7) * 128 + ((((byte >> 4) ^ (linha & 7)) << 4) | (byte & 15)));
}
__device__ __forceinline__ void fence_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// 16 columns of this thread's lane from three accumulators `passo` columns apart (hi.hi, cross, lo.lo)
__device__ __forceinline__ void tmem_le16x3(uint32_t t, uint32_t (&a)[16], uint32_t (&b)[16], uint32_t (&c)[16], uint32_t passo = NI) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%48];\n"
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%49];\n"
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%32,%33,%34,%35,%36,%37,%38,%39,%40,%41,%42,%43,%44,%45,%46,%47}, [%50];\n"
        "tcgen05.wait::ld.sync.aligned;\n"
        : JT_O16(a, 0), JT_O16(b, 0), JT_O16(c, 0)
        : "r"(t), "r"(t + passo), "r"(t + 2 * passo)
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
// the four MMAs of one score-like product: A = 128 rows of [hi | lo], B = the stacked query tile (3 NI rows) -> hi.hi | cross | lo.lo
__device__ __forceinline__ void mma_digitos(uint32_t tm, uint64_t da, uint64_t db3) {
#pragma unroll
    for (int q = 0; q < 4; q++) tc_mma_i8(tm, da + 2 * q, db3 + 2 * q, ID_S3, q != 0);
}
// the stacked B operand from a tile of NI rows of [hi | lo] (128-byte swizzle on both sides): rows 0..NI-1 = [hi | 0],
// NI..2NI-1 = [lo | hi], 2NI..3NI-1 = [0 | lo].  Called by all NTL threads; 16-byte pieces.
__device__ __forceinline__ void empilha3(const unsigned char* orig, unsigned char* dest, int tid) {
    for (int t = tid; t < 3 * NI * 8; t += NTL) {
        const int R = t >> 3, c = t & 7, bloco = R / NI, r = R % NI;
        int co = -1;                                               // source piece, -1 = zeros
        if (bloco == 0) co = c < 4 ? c : -1;
        else if (bloco == 1) co = c < 4 ? c + 4 : c - 4;
        else co = c < 4 ? -1 : c;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (co >= 0) v = *reinterpret_cast<const uint4*>(orig + (r >> 3) * 1024 + (r & 7) * 128 + ((co ^ (r & 7)) << 4));
        *reinterpret_cast<uint4*>(dest + (R >> 3) * 1024 + (R & 7) * 128 + ((c ^ (R & 7)) << 4)) = v;
    }
}
// CTA-wide maximum of a non-negative per-thread value (NTL threads) -> one atomicMax
__device__ __forceinline__ void max_cta16(int v, int* destino, int* red, int tid) {
    v = warp_max(v);
    __syncthreads();
    if ((tid & 31) == 0) red[tid >> 5] = v;
    __syncthreads();
    if (tid == 0) {
        int r = red[0];
#pragma unroll
        for (int i = 1; i < NTL / 32; i++) r = max(r, red[i]);
        if (r > 0) atomicMax(destino, r);
    }
}
__device__ __forceinline__ int junta3(uint32_t hh, uint32_t cr, uint32_t ll) { return (int)((hh << 14) + (cr << 7) + ll); }

// Output of 8 consecutive columns of one row (the 4 lanes tid & 3 = 0..3 hold the 32 columns of one exponent block, all with the
// exponent e): raw (int32 + int16 exponent per element), or - the caller asked for the quantised form and the block length is 32 -
// straight to a block tensor, i.e. jt_quant of the raw output (ops.py:125-126) without the round trip through memory.
// All 32 lanes of a warp call it together (the quantiser shuffles); `grava` = false computes and stores nothing.
__device__ __forceinline__ void grava8(int* acc, int16_t* ex, int8_t* qm, int8_t* qE, size_t p, size_t pe, const int (&o)[8], int e, int kid, int tid,
                                       bool grava = true) {
    if (qm) {
        int q[8];
        const int E = quant_uniforme<8, 4>(o, e, q, kid, (long long)p);
        if (!grava) return;
        *reinterpret_cast<uint2*>(qm + p) = make_uint2(junta4(q[0], q[1], q[2], q[3]), junta4(q[4], q[5], q[6], q[7]));
        if ((tid & 3) == 0) qE[pe] = (int8_t)E;
        return;
    }
    if (!grava) return;
    const uint32_t e2 = (uint32_t)(e & 0xffff) | ((uint32_t)e << 16);
    *reinterpret_cast<int4*>(acc + p) = make_int4(o[0], o[1], o[2], o[3]);
    *reinterpret_cast<int4*>(acc + p + 4) = make_int4(o[4], o[5], o[6], o[7]);
    *reinterpret_cast<uint4*>(ex + p) = make_uint4(e2, e2, e2, e2);
}

// -------------------------------------------------------------------------------------------------- preparation
// z = 0 q, 1 k, 2 v (columns of QKV), 3 dO.  Per tensor: destination in row layout and / or transposed layout (nullptr = not needed).
struct ArgsPrep {
    const int8_t* qm; const int8_t* qE; const int8_t* gm; const int8_t* gE;
    int8_t* lin[4]; int8_t* tra[4];
    int* em;                    // [BH][4] head-maximum exponents, indexed by z
    int* est;                   // backward: the statistics slots [BH][N_EST] to clear (nullptr in the forward)
    int* nrm;                   // forward: [BH][2][ceil(T/128)] largest sum of squares of an aligned row of q (0) / k (1) per 128 tokens, or nullptr
    int T, H, D, GA, blk;
};

// grid (ceil(T / 128), BH, 4), 256 threads: 128 tokens of one head of one tensor
__global__ void __launch_bounds__(256) k_at_prep(const ArgsPrep A) {
    pdl_espera();
    pdl_solta();
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
    if (A.est && blockIdx.x == 0 && z == 3 && tid < at::N_EST) A.est[bh * at::N_EST + tid] = 0;
    const int r = tid >> 1, meio = tid & 1, t = t0 + r;
    int norma = 0;
    if (t < T) {
        const size_t lin = (size_t)(linha0 + t);
#pragma unroll
        for (int parte = 0; parte < 2; parte++) {
            const int c = meio * 32 + parte * 16;
            int v[16], hi[16], lo[16];
            le16(m + lin * ld + col0 + c, v);
            const int s = em - (int)E[lin * ldb + (col0 + c) / blk];
#pragma unroll
            for (int k = 0; k < 16; k++) {
                const int a = rnd_d(v[k] << A.GA, s);
                norma += a * a;                                    // 12-bit values, 64 of them: below 2^28
                digitos(a, hi[k], lo[k]);
            }
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
    if (A.nrm && z < 2) {
        // the largest squared norm of an aligned row among this CTA's 128 tokens (the two halves of a row sit in neighbouring lanes)
        norma += __shfl_xor_sync(0xffffffffu, norma, 1);
        norma = __reduce_max_sync(0xffffffffu, norma);
        __syncthreads();                                           // red[] is free again (max_cabeca used it)
        if ((tid & 31) == 0) red[tid >> 5] = norma;
        __syncthreads();
        if (tid == 0) {
            int mx = 0;
            for (int w = 0; w < 8; w++) mx = max(mx, red[w]);
            A.nrm[((size_t)bh * 2 + z) * gridDim.x + blockIdx.x] = mx;
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
// ops.py:198-219.  grid (T / 64, BH), 512 threads; a drain thread owns one key of the chunk and 16 of the 64 query rows.
//   sweep 1 over the key chunks: scores u (tensor core + drain), row maxima;
//   sweep 2: the scores again (recomputing costs 13 instructions per score, keeping them 128 KB of shared memory), the
//            exponentials ex = exp(-(m - u)/256) >> 3 (12 bits, kept as uint16 [64][T+8]) and their row sums;
//   pass 3 : P = min((ex * inv + 2^19) >> 20, 255); the thread's 16 rows of its key are 16 contiguous bytes of the stored,
//            key-major P; the same bytes go to a small MMA-layout tile and O^T += V^T . P^T runs chunk by chunk behind it.
// Shared: 2 operand stages (K chunks, then V^T chunks), the query tile as loaded and stacked, 2 P tiles, ex.  Tensor memory:
// two score buffers of 3 x 64 columns, one output accumulator of 64 columns (512 allocated, one CTA per SM).
__global__ void __launch_bounds__(NTL) k_atencao_tc(const __grid_constant__ CUtensorMap mQ, const __grid_constant__ CUtensorMap mK,
                                                    const __grid_constant__ CUtensorMap mVt, const int* __restrict__ em, int* __restrict__ Oacc,
                                                    int16_t* __restrict__ Oe, int8_t* __restrict__ Qm, int8_t* __restrict__ QE, uint8_t* __restrict__ P,
                                                    int T, int H, int D, int GA, int kid) {
    extern __shared__ unsigned char bruto[];
    // (pointer arithmetic on the array keeps the shared address space: a round trip through an integer makes every access generic)
    unsigned char* smem = bruto + ((1024u - (smem_u32(bruto) & 1023u)) & 1023u);
    const uint32_t sbase = smem_u32(smem);
    const int nchT = (T + TJ - 1) / TJ, TPX = T + 8;
    // 3 operand stages (a TMA load takes longer than one step of a sweep: loads run three steps ahead) | stacked query tile |
    // 2 P tiles (the query tile as loaded sits there until it has been stacked) | barriers, row statistics | ex
    constexpr int NSTF = 3;
    constexpr uint32_t OFF_Q3 = NSTF * TILE_A, OFF_PB = OFF_Q3 + TILE_Q3, OFF_Q = OFF_PB, OFF_BAR = OFF_PB + 2 * TILE_NI, OFF_EX = OFF_BAR + 640;
    uint8_t* pB = smem + OFF_PB;                                   // [2][64 x 128]
    uint16_t* ex_s = reinterpret_cast<uint16_t*>(smem + OFF_EX);   // [64][T + 8]
    const Barras bar = {sbase + OFF_BAR};                          // 0 q | 1..3 k | 4,5 s | 6..8 v | 9,10 pv done | 11 o
    constexpr int B_K = 1, B_S = 4, B_V = 6, B_PV = 9, B_O = 11;
    uint32_t* slot = reinterpret_cast<uint32_t*>(smem + OFF_BAR + 112);
    volatile int* aborta = reinterpret_cast<volatile int*>(smem + OFF_BAR + 116);
    int* m_s = reinterpret_cast<int*>(smem + OFF_BAR + 128);       // [64] row maxima, then 2^28 / row sum
    int* s_acc = m_s + NI;                                         // [64] row sums
    const int tid = threadIdx.x, wid = tid >> 5, lane = tid & 31;
    const int ordem = blockIdx.y * gridDim.x + blockIdx.x;         // heaviest (last) row tiles of all heads first
    const int bh = ordem % gridDim.y, b = bh / H, h = bh % H, i0 = (gridDim.x - 1 - ordem / gridDim.y) * NI, linha0 = b * T;
    const int nproc = i0 + NI, nch = (nproc + TJ - 1) / TJ;
    const uint32_t sA[NSTF] = {sbase, sbase + TILE_A, sbase + 2 * TILE_A}, sQ = sbase + OFF_Q, sQ3 = sbase + OFF_Q3, sPB = sbase + OFF_PB;
    // a CTA lives a few microseconds, so what it waits for first is asked for first: the operand loads go out as soon as their
    // barriers exist, the small global reads follow, and tensor memory is allocated while all of that is in flight
    if (tid == 0) {
        for (int i = 0; i < 12; i++) mbar_init(bar[i], 1);
        *aborta = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    pdl_espera();                                                  // the operands below are the previous kernel's outputs
    pdl_solta();
    const bool pode_pular = T > 2 * TJ;                            // up to two key chunks nearly every chunk is next to the diagonal
    if (tid == 0) {
        mbar_expect_tx(bar[0], TILE_NI);
        tma_2d(sQ, &mQ, 0, bh * T + i0, bar[0]);
        if (!pode_pular)                                           // every chunk stays: its loads need not wait for the bound
            for (int c = 0; c < NSTF && c < 2 * nch; c++) {
                mbar_expect_tx(bar[B_K + c], TILE_A);
                tma_2d(sA[c], &mK, 0, bh * T + (c % nch) * TJ, bar[B_K + c]);
            }
    }
    const int emq = em[bh * 4], emk = em[bh * 4 + 1], emv = em[bh * 4 + 2];
    const int s_u = -((emq - GA) + (emk - GA) - 3 + 8), incl = at::incl_alibi(h);
    // Key chunks that cannot matter.  |q_i . k_j| <= sqrt(|q_i|^2 |k_j|^2) (the preparation left the largest squared norms per 128
    // tokens), so with B >= (|x| >> s_u) + 1 every score is u_ij <= B - (i - j) 2^incl and every row maximum is m_i >= u_ii >= -B.
    // The exponential (>> 3) is exactly 0 from m - u = 2130 on (p < 2^15 shifted by n + 3 >= 15), so a key at distance
    // (i - j) 2^incl >= 2132 + 2 B adds nothing to the row sum, cannot be the maximum and has P = 0: chunks wholly at that distance
    // from the tile's first query are left out of all three passes (P = 0 is still written).  Only on the right-shift path.
    int c0 = 0;
    if (pode_pular && s_u > 0 && s_u < 31) {
        const int* nrm = em + 4 * gridDim.y;
        const int nq = nrm[((size_t)bh * 2) * nchT + i0 / TJ];
        int nk = 0;
        for (int c = 0; c < nch; c++) nk = max(nk, nrm[((size_t)bh * 2 + 1) * nchT + c]);
        const long long B = ((long long)sqrt((double)nq * (double)nk) + 2) >> s_u;
        const long long lim = 2132 + 2 * (B + 2), D0 = (lim + (1 << incl) - 1) >> incl;
        if (i0 - D0 + 1 > 0) c0 = (int)((i0 - D0 + 1) / TJ);
    }
    const int nviv = nch - c0, nvoltas = 2 * nviv;                  // live chunks c0 .. nch - 1, swept twice
    if (tid == 0 && pode_pular) {
        for (int c = 0; c < NSTF && c < nvoltas; c++) {
            mbar_expect_tx(bar[B_K + c], TILE_A);
            tma_2d(sA[c], &mK, 0, bh * T + (c0 + c % nviv) * TJ, bar[B_K + c]);
        }
    }
    if (tid < NI) { m_s[tid] = U_MIN; s_acc[tid] = 0; }
    if (wid == 0) tmem_aloca(slot, 512);
    tc_fence_antes();
    __syncthreads();
    tc_fence_depois();
    const uint32_t tmem = *slot;
    const int jl = 32 * (wid & 3) + lane, g = wid >> 2;            // this thread's key within a chunk, its quarter of the query rows
    const uint32_t t_lane = tmem + ((uint32_t)(32 * (wid & 3)) << 16);

    auto emite = [&](int cc) -> bool {                             // one thread: the score MMAs of step cc (key chunk cc % nch)
        if (!espera(bar[B_K + cc % NSTF], (cc / NSTF) & 1, aborta, kid, 21)) return false;
        tc_fence_depois();
        mma_digitos(tmem + (cc & 1) * SB, desc_sw128(sA[cc % NSTF]), desc_sw128(sQ3));
        tc_commit(bar[B_S + (cc & 1)]);
        return true;
    };
    int v16[16], mi[16];                                           // running maxima, then running sums | this thread's row maxima, then 2^28 / sum
#pragma unroll
    for (int k = 0; k < 16; k++) { v16[k] = U_MIN; mi[k] = 0; }
    bool ok = __all_sync(FULL, espera(bar[0], 0, aborta, kid, 20));     // the query tile has landed: stack its three arrangements
    if (ok) empilha3(smem + OFF_Q, smem + OFF_Q3, tid);
    fence_async();
    __syncthreads();
    if (tid == 0 && ok) ok = emite(0);
    for (int cc = 0; cc < nvoltas; cc++) {
        const int c = c0 + cc % nviv, st = cc & 1;
        if (tid == 0 && ok && cc + 1 < nvoltas) ok = emite(cc + 1);
        __syncwarp();
        ok = __all_sync(FULL, ok && espera(bar[B_S + st], (cc >> 1) & 1, aborta, kid, 22));
        tc_fence_depois();
        if (tid == 0 && ok && cc + NSTF < nvoltas) {               // this step's MMAs are done: its stage takes the chunk of step cc + 3
            mbar_expect_tx(bar[B_K + cc % NSTF], TILE_A);
            tma_2d(sA[cc % NSTF], &mK, 0, bh * T + (c0 + (cc + NSTF) % nviv) * TJ, bar[B_K + cc % NSTF]);
        }
        if (cc == nviv) {
            // between the sweeps: the row maxima from the per-thread maxima
#pragma unroll
            for (int k = 0; k < 16; k++) {
                const int m = warp_max(v16[k]);
                if (lane == 0) atomicMax(&m_s[16 * g + k], m);
            }
            __syncthreads();
#pragma unroll
            for (int k = 0; k < 16; k++) { mi[k] = m_s[16 * g + k]; v16[k] = 0; }
        }
        if (ok) {
            const int j = c * TJ + jl;
            uint32_t hh[16], cr[16], ll[16];
            tmem_le16x3(t_lane + st * SB + 16 * g, hh, cr, ll);
            if (j < nproc && s_u > 0 && s_u < 31) {
                // the usual case, a right shift: rounding, slope and exponential written out with their invariants hoisted.
                //   rnd_d(x, s)              = (x + 2^(s-1) - 1 + ((x >> s) & 1)) >> s
                //   exp_int(d) >> 3, d>=0    : t = min(d, 6000) * 23637, n = t >> 22, f = bits 7..21 of t; the cubic in f runs on
                //                              p * 2^16 (|p| < 2^15 at every step): (p f) >> 15 = mulhi(p << 16, 2 f); the result
                //                              p >> (n + 3) is 0 from n = 12 on (0 <= p < 2^15), as is the shift clamped to 31
                const int meio = (1 << (s_u - 1)) - 1, dj = i0 + 16 * g - j, menos = -(1 << incl);
                const bool diagonal = c == nch - 1;                    // the only chunk with keys beyond some query of the tile
#pragma unroll
                for (int k = 0; k < 16; k++) {
                    const int x = junta3(hh[k], cr[k], ll[k]);
                    int u = (x + meio + ((x >> s_u) & 1)) >> s_u;
                    u += (dj + k) * menos;
                    const bool dentro = !diagonal || dj + k >= 0;
                    if (cc < nviv) v16[k] = max(v16[k], dentro ? u : U_MIN);
                    else {
                        // a key beyond the diagonal counts as infinitely far below the maximum; mi >= u otherwise, and
                        // |u| < 2^30 + 2^18: the difference cannot overflow
                        const int t = min(dentro ? mi[k] - u : 6000, 6000) * 23637;
                        const int f2 = (t >> 6) & 0xFFFE;
                        int pp = -1295 * 65536;
                        pp = __mulhi(pp, f2) * 65536 + 7556 * 65536;
                        pp = __mulhi(pp, f2) * 65536 - 22645 * 65536;
                        pp = __mulhi(pp, f2) * 65536 + 32765 * 65536;
                        const int ex = pp >> min(19 + (t >> 22), 31);
                        v16[k] += ex;
                        ex_s[(16 * g + k) * TPX + j] = (uint16_t)ex;
                    }
                }
            } else if (j < nproc) {
#pragma unroll
                for (int k = 0; k < 16; k++) {
                    const int i = i0 + 16 * g + k;
                    const bool dentro = j <= i;
                    int u = U_MIN;
                    if (dentro) u = rnd(junta3(hh[k], cr[k], ll[k]), s_u, kid, (long long)(linha0 + i) * D + h * HD) - ((i - j) << incl);
                    if (cc < nviv) v16[k] = max(v16[k], u);
                    else {
                        const int ex = dentro ? exp_dif(mi[k], u) >> 3 : 0;
                        v16[k] += ex;
                        ex_s[(16 * g + k) * TPX + j] = (uint16_t)ex;
                    }
                }
            }
        }
        tc_fence_antes();
        __syncthreads();
    }
    // row sums -> 2^28 / sum (ops.py:215)
#pragma unroll
    for (int k = 0; k < 16; k++) {
        const int sm = warp_sum(v16[k]);
        if (lane == 0) atomicAdd(&s_acc[16 * g + k], sm);
    }
    __syncthreads();
    if (tid < NI) {
        int soma = s_acc[tid];
        if (soma <= 0) { reporta(E_DIV, kid, (long long)(linha0 + i0 + tid) * D + h * HD, soma, 0); soma = 1; }
        m_s[tid] = (1 << 28) / soma;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < 16; k++) mi[k] = m_s[16 * g + k];
    // pass 3: P of every key (explicit zeros before the first live chunk and beyond the diagonal, to the end of the sequence) and
    // O^T += V^T . P^T behind it, over the live chunks (m = c - c0 counts them: stages and parities go by m)
    if (tid == 0 && ok) {
        for (int m = 0; m < NSTF && m < nviv; m++) {
            mbar_expect_tx(bar[B_V + m], TILE_A);
            tma_2d(sA[m], &mVt, (c0 + m) * TJ, bh * 128, bar[B_V + m]);
        }
    }
    for (int c = 0; c < nchT; c++) {
        const int m = c - c0, st = m & 1, j = c * TJ + jl;
        const bool com_mma = c >= c0 && c < nch;
        if (com_mma && m >= 2) ok = __all_sync(FULL, ok && espera(bar[B_PV + st], ((m - 2) >> 1) & 1, aborta, kid, 26));      // tile st is free again
        if (com_mma && m >= 2 && m + 1 >= NSTF && m + 1 < nviv && tid == 0 && ok) {      // and so is the operand stage of chunk m - 2: it takes chunk m + 1
            mbar_expect_tx(bar[B_V + (m + 1) % NSTF], TILE_A);
            tma_2d(sA[(m + 1) % NSTF], &mVt, (c + 1) * TJ, bh * 128, bar[B_V + (m + 1) % NSTF]);
        }
        uint32_t w[4] = {0, 0, 0, 0};
        if (com_mma && j < nproc) {
#pragma unroll
            for (int k = 0; k < 16; k++) {
                const int p = min(((int)ex_s[(16 * g + k) * TPX + j] * mi[k] + (1 << 19)) >> 20, 255);
                w[k >> 2] |= (uint32_t)p << (8 * (k & 3));
            }
        }
        if (j < T) *reinterpret_cast<uint4*>(P + ((size_t)bh * T + j) * T + i0 + 16 * g) = make_uint4(w[0], w[1], w[2], w[3]);
        if (!com_mma) continue;
#pragma unroll
        for (int k = 0; k < 16; k++) pB[st * TILE_NI + sw128(16 * g + k, jl)] = (uint8_t)(w[k >> 2] >> (8 * (k & 3)));
        fence_async();                                             // the tile is read by the tensor core (async proxy)
        __syncthreads();
        if (tid == 0 && ok) {
            ok = espera(bar[B_V + m % NSTF], (m / NSTF) & 1, aborta, kid, 23);
            if (ok) {
                tc_fence_depois();
                const uint64_t da = desc_sw128(sA[m % NSTF]), db = desc_sw128(sPB + st * TILE_NI);
#pragma unroll
                for (int q = 0; q < 4; q++) tc_mma_i8(tmem + 2 * SB, da + 2 * q, db + 2 * q, ID_PU, (m | q) != 0);
                tc_commit(bar[B_PV + st]);
                if (c == nch - 1) tc_commit(bar[B_O]);
            }
        }
    }
    __syncwarp();
    ok = __all_sync(FULL, ok && espera(bar[B_O], 0, aborta, kid, 25));
    tc_fence_depois();
    __syncthreads();                                               // every thread is done with ex_s: it becomes the staging area
    int* o_s = reinterpret_cast<int*>(smem + OFF_EX);              // [128 digit rows][65]
    if (ok) {
        uint32_t d[16];
        tmem_le16(t_lane + 2 * SB + 16 * g, d);
#pragma unroll
        for (int k = 0; k < 16; k++) o_s[jl * 65 + 16 * g + k] = (int)d[k];
    }
    tc_fence_antes();
    __syncthreads();
    {
        const int i = tid >> 3, d0 = (tid & 7) * 8;
        int o[8];
#pragma unroll
        for (int k = 0; k < 8; k++) o[k] = (int)(((uint32_t)o_s[(d0 + k) * 65 + i] << 7) + (uint32_t)o_s[(64 + d0 + k) * 65 + i]);
        const size_t lin = (size_t)(linha0 + i0 + i);
        grava8(Oacc, Oe, Qm, QE, lin * D + h * HD + d0, lin * (D / 32) + (h * HD + d0) / 32, o, (emv - GA) - 8, kid, tid);
    }
    if (wid == 0) {
        tc_fence_depois();
        tmem_libera(tmem, 512);
    }
}
// ex needs 64 * (T + 8) * 2 bytes, the output staging that reuses it 128 * 65 * 4
inline size_t smem_frente_tc(int T) {
    const size_t ex = (size_t)NI * (T + 8) * 2, os = 128 * 65 * 4;
    return 1024 + 3 * TILE_A + TILE_Q3 + 2 * TILE_NI + 640 + (ex > os ? ex : os);
}

// -------------------------------------------------------------------------------------------------- where stored P is zero
// zm[bh][kt] = bit qt set when P (key-major, [BH*T][T]) has a non-zero among keys 64 kt .. 64 kt + 63 and queries 64 qt .. 64 qt + 63.
// grid (ceil(T / 64), BH), 256 threads: 4 threads per key row, from the diagonal on (P is zero above it by construction).
__global__ void __launch_bounds__(256) k_p_mapa(const uint8_t* __restrict__ P, int* __restrict__ zm, int T) {
    pdl_espera();
    pdl_solta();
    __shared__ unsigned ou;
    const int tid = threadIdx.x, kt = blockIdx.x, bh = blockIdx.y, r = tid >> 2, parte = tid & 3, j = kt * NJ + r;
    if (tid == 0) ou = 0;
    __syncthreads();
    unsigned m = 0;
    if (j < T) {
        const uint4* linha = reinterpret_cast<const uint4*>(P + ((size_t)bh * T + j) * T);
        for (int p = 4 * kt + parte; p < T / 16; p += 4) {          // 16-byte pieces; piece p belongs to query tile p / 4
            const uint4 v = linha[p];
            if (v.x | v.y | v.z | v.w) m |= 1u << (p >> 2);
        }
    }
    m = __reduce_or_sync(0xffffffffu, m);
    if ((tid & 31) == 0 && m) atomicOr(&ou, m);
    __syncthreads();
    if (tid == 0) zm[bh * gridDim.x + kt] = (int)ou;
}

// -------------------------------------------------------------------------------------------------- backward, row tiles
struct ArgsTrasTC {
    const uint8_t* P; int* Gacc; int16_t* Ge; int* est; int* sl; const int* em;      // em: [BH][4] = q, k, v, dO
    const int* zm;                                                                    // [BH][ceil(T/64)]: per 64 keys, bit qt = P has a non-zero among queries 64 qt .. 64 qt + 63
    int8_t* DSh; int8_t* DSl;                                                         // [BH*T][T] digits of dS', key-major (transposed)
    int8_t* Gm; int8_t* GE;                                                           // block output [M, 3D] instead of the raw one, or nullptr
    int T, H, D, GA, limite, kid;
};

// FASE 1: max |gP| over j <= i.   FASE 2: s_lin and the maxima of dS (two sweeps over the keys).   FASE 3: dS' (digits to the
// workspace, key-major, for the key-tile kernel) and gq = dS' . k.     grid (T / 64, BH), 512 threads.
// Every sweep recomputes gP = dO . v^T on the tensor core; nothing T x T is kept in shared memory.
// Tensor memory: two score buffers (3 x 64 columns each) + in phase 3 two output accumulators of 64 columns (512 allocated).
template <int FASE>
__global__ void __launch_bounds__(NTL) k_ab_linhas_tc(const __grid_constant__ CUtensorMap mV, const __grid_constant__ CUtensorMap mG,
                                                      const __grid_constant__ CUtensorMap mKt, const ArgsTrasTC A) {
    extern __shared__ unsigned char bruto[];
    // (pointer arithmetic on the array keeps the shared address space: a round trip through an integer makes every access generic)
    unsigned char* smem = bruto + ((1024u - (smem_u32(bruto) & 1023u)) & 1023u);
    const uint32_t sbase = smem_u32(smem);
    // stages: V chunks [4] (a TMA load takes longer than a step of a sweep: loads run four steps ahead) | dO tile as loaded |
    // dO tile stacked | (phase 3) K^T chunks [4] | dS' digit tiles [2][hi rows, lo rows]
    constexpr int NSTV = 4;
    constexpr uint32_t OFF_G = NSTV * TILE_A, OFF_G3 = OFF_G + TILE_NI, OFF_KT = OFF_G3 + TILE_Q3, OFF_DS = OFF_KT + (FASE == 3 ? NSTV * TILE_A : 0);
    constexpr uint32_t OFF_BAR = OFF_DS + (FASE == 3 ? 4 * TILE_NI : 0);
    const Barras bar = {sbase + OFF_BAR};                          // 0 dO | 1..4 v | 5,6 s | 7..10 kt | 11,12 gq done | 13 o
    constexpr int B_V = 1, B_S = 5, B_KT = 7, B_G = 11, B_O = 13;
    uint32_t* slot = reinterpret_cast<uint32_t*>(smem + OFF_BAR + 112);
    volatile int* aborta = reinterpret_cast<volatile int*>(smem + OFF_BAR + 116);
    int* sl_s = reinterpret_cast<int*>(smem + OFF_BAR + 128);      // [64]
    int* s_acc = sl_s + NI;                                        // [64]
    __shared__ int red[NTL / 32];
    const int T = A.T, H = A.H, D = A.D, GA = A.GA, kid = A.kid;
    const int tid = threadIdx.x, wid = tid >> 5, lane = tid & 31;
    const int ordem = blockIdx.y * gridDim.x + blockIdx.x;
    const int bh = ordem % gridDim.y, b = bh / H, h = bh % H, i0 = (gridDim.x - 1 - ordem / gridDim.y) * NI, linha0 = b * T;
    int* est = A.est + bh * at::N_EST;
    const int nproc = i0 + NI, nch = (nproc + TJ - 1) / TJ;
    const uint32_t sG = sbase + OFF_G, sG3 = sbase + OFF_G3, sKt0 = sbase + OFF_KT;          // V stage s at sbase + s * TILE_A, K^T stage s at sKt0 + s * TILE_A
    uint8_t* ds_b = smem + OFF_DS;                                 // [2 stages][hi rows | lo rows][64 x 128]
    // first the operand loads (as soon as their barriers exist), then the small global reads, then tensor memory
    if (tid == 0) {
        for (int i = 0; i < 14; i++) mbar_init(bar[i], 1);
        *aborta = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    pdl_espera();                                                  // the operands below are the previous kernel's outputs
    pdl_solta();
    if (tid == 0) {
        mbar_expect_tx(bar[0], TILE_NI);
        tma_2d(sG, &mG, 0, bh * T + i0, bar[0]);
    }
    // Key chunks in which stored P is zero for this query tile and its two neighbours (A.zm: per 64 keys, the 64-query tiles
    // with a non-zero P) add nothing to s_lin, dS' and gq, and the key-tile kernel does not read their dS': phases 2 and 3 leave
    // them out.  The diagonal chunk always stays; phase 1 (a maximum over every position) and the bounded variant keep them all.
    unsigned vivos = (1u << nch) - 1u;
    if (FASE != 1 && !A.limite && A.zm) {
        const int qt = i0 / NI, nkt = (T + NJ - 1) / NJ;
        const unsigned vizinhos = (7u << qt) >> 1;                 // query tiles qt - 1, qt, qt + 1
        vivos = 1u << (nch - 1);
        if (qt >= 1) vivos |= 1u << ((qt - 1) / 2);               // the chunk of key tile qt - 1: the key-tile kernel's first step reads it
        for (int c = 0; c < nch - 1; c++) {
            unsigned m = (unsigned)A.zm[bh * nkt + 2 * c];
            if (2 * c + 1 < nkt) m |= (unsigned)A.zm[bh * nkt + 2 * c + 1];
            if (m & vizinhos) vivos |= 1u << c;
        }
    }
    const int nviv = __popc(vivos);
    const int nvoltas = FASE == 2 ? 2 * nviv : nviv;               // phase 2 sweeps the keys twice
    auto pedaco = [&](int cc) -> int { return (int)__fns(vivos, 0, cc % nviv + 1); };      // the live chunk of step cc
    if (tid == 0) {
        for (int c = 0; c < NSTV && c < nvoltas; c++) {
            mbar_expect_tx(bar[B_V + c], TILE_A);
            tma_2d(sbase + c * TILE_A, &mV, 0, bh * T + pedaco(c) * TJ, bar[B_V + c]);
        }
        if (FASE == 3)
            for (int c = 0; c < 2 && c < nviv; c++) {
                mbar_expect_tx(bar[B_KT + c], TILE_A);
                tma_2d(sKt0 + c * TILE_A, &mKt, pedaco(c) * TJ, bh * 128, bar[B_KT + c]);
            }
    }
    const int emk = A.em[bh * 4 + 1], emv = A.em[bh * 4 + 2], emg = A.em[bh * 4 + 3];
    const int sh = FASE == 1 ? 0 : at::desl1(est, A.limite);
    const int sh2 = FASE == 3 ? at::desl2(est, A.limite) : 0;
    if (tid < NI) { s_acc[tid] = 0; sl_s[tid] = FASE == 3 ? A.sl[(size_t)bh * T + i0 + tid] : 0; }
    if (wid == 0) tmem_aloca(slot, 512);
    tc_fence_antes();
    __syncthreads();
    tc_fence_depois();
    const uint32_t tmem = *slot;
    const int nzero = min((nproc + NJ - 1) / NJ * NJ, T);          // phase 3 writes explicit zeros of dS' up to the key tile's end
    auto emite = [&](int cc) -> bool {
        if (!espera(bar[B_V + cc % NSTV], (cc / NSTV) & 1, aborta, kid, 31)) return false;
        tc_fence_depois();
        mma_digitos(tmem + (cc & 1) * SB, desc_sw128(sbase + (cc % NSTV) * TILE_A), desc_sw128(sG3));
        tc_commit(bar[B_S + (cc & 1)]);
        return true;
    };
    int mgp = 0, mds = 0, mp = 0;
    int s_part[16];
#pragma unroll
    for (int k = 0; k < 16; k++) s_part[k] = 0;
    bool ok = __all_sync(FULL, espera(bar[0], 0, aborta, kid, 30));     // the dO tile has landed: stack its three arrangements
    if (ok) empilha3(smem + OFF_G, smem + OFF_G3, tid);
    fence_async();
    __syncthreads();
    if (tid == 0 && ok) ok = emite(0);
    for (int cc = 0; cc < nvoltas; cc++) {
        const int c = pedaco(cc), st = cc & 1;
        if (tid == 0 && ok && cc + 1 < nvoltas) ok = emite(cc + 1);
        __syncwarp();
        ok = __all_sync(FULL, ok && espera(bar[B_S + st], (cc >> 1) & 1, aborta, kid, 32));
        tc_fence_depois();
        if (tid == 0 && ok && cc + NSTV < nvoltas) {               // this step's MMAs are done: its stage takes the chunk of step cc + 4
            mbar_expect_tx(bar[B_V + cc % NSTV], TILE_A);
            tma_2d(sbase + (cc % NSTV) * TILE_A, &mV, 0, bh * T + pedaco(cc + NSTV) * TJ, bar[B_V + cc % NSTV]);
        }
        if (FASE == 3) {
            // the digit tiles of this parity and the K^T stage of chunk cc - 2 are free once that chunk's output MMAs are done;
            // the stage takes chunk cc + 2 (the first two steps fill the stages nobody has used yet)
            if (cc >= 2) ok = __all_sync(FULL, ok && espera(bar[B_G + st], ((cc - 2) >> 1) & 1, aborta, kid, 33));
            if (tid == 0 && ok && cc + 2 < nviv) {
                mbar_expect_tx(bar[B_KT + (cc + 2) % NSTV], TILE_A);
                tma_2d(sKt0 + ((cc + 2) % NSTV) * TILE_A, &mKt, pedaco(cc + 2) * TJ, bh * 128, bar[B_KT + (cc + 2) % NSTV]);
            }
        }
        if (FASE == 2 && cc == nviv) {
            // between the sweeps: s_lin of the 32 rows from the per-thread partial sums
#pragma unroll
            for (int k = 0; k < 16; k++) {
                const int s = warp_sum(s_part[k]);
                if (lane == 0) atomicAdd(&s_acc[16 * (wid >> 2) + k], s);
            }
            __syncthreads();
            if (tid < NI) {
                const int sl = rnd_d(s_acc[tid], 8);
                sl_s[tid] = sl;
                A.sl[(size_t)bh * T + i0 + tid] = sl;
            }
            __syncthreads();
        }
        if (ok) {
            const int jl = 32 * (wid & 3) + lane, g = wid >> 2, j = c * TJ + jl;
            uint32_t hh[16], cr[16], ll[16];
            tmem_le16x3(tmem + ((uint32_t)(32 * (wid & 3)) << 16) + st * SB + 16 * g, hh, cr, ll);
            uint32_t pw[4] = {0, 0, 0, 0};
            if (FASE != 1 && j < nproc) {
                const uint4 w = *reinterpret_cast<const uint4*>(A.P + ((size_t)bh * T + j) * T + i0 + 16 * g);
                pw[0] = w.x; pw[1] = w.y; pw[2] = w.z; pw[3] = w.w;
            }
            int dh[16], dl[16];
            // A key counts for query i0 + 16 g + k when it exists for this tile (j < nproc) and is not beyond the diagonal, which only
            // the last chunk can be: one comparison of k against a per-thread bound.  With both shifts in 1..30 the roundings are
            // written out with their constants hoisted: rnd_d(x, s) = (x + 2^(s-1) - 1 + ((x >> s) & 1)) >> s.
            const int kmin = j >= nproc ? 16 : (c == nch - 1 ? j - (i0 + 16 * g) : 0);      // dentro <=> k >= kmin
            auto corpo = [&](auto rapido_t) {
                constexpr bool RAP = decltype(rapido_t)::value;
                const int meio1 = RAP && FASE != 1 ? (1 << max(sh - 1, 0)) - 1 : 0, meio2 = RAP && FASE == 3 ? (1 << max(sh2 - 1, 0)) - 1 : 0;
#pragma unroll
                for (int k = 0; k < 16; k++) {
                    const bool dentro = k >= kmin;
                    const int x = junta3(hh[k], cr[k], ll[k]);
                    int gp;
                    if (FASE == 1) gp = x;
                    else if (RAP) gp = (x + meio1 + ((x >> sh) & 1)) >> sh;
                    else gp = rnd_d(x, sh);
                    gp = dentro ? gp : 0;
                    if (FASE == 1 || (FASE == 2 && cc < nviv)) mgp = max(mgp, gp < 0 ? -gp : gp);
                    if (FASE == 1) continue;
                    const int p = (int)((pw[k >> 2] >> (8 * (k & 3))) & 0xff);
                    if (FASE == 2) {
                        if (cc < nviv) s_part[k] += p * gp;
                        else {
                            const int ds = p * (gp - sl_s[16 * g + k]);
                            mds = max(mds, ds < 0 ? -ds : ds);
                            mp = max(mp, p);
                        }
                    } else {
                        const int y = p * (gp - sl_s[16 * g + k]);
                        int ds;
                        if (RAP) ds = (y + meio2 + ((y >> sh2) & 1)) >> sh2;
                        else ds = rnd_d(y, sh2);
                        ds = dentro ? ds : 0;
                        digitos(ds, dh[k], dl[k]);
                        ds_b[(2 * st) * TILE_NI + sw128(16 * g + k, jl)] = (uint8_t)dh[k];              // rows 0..63 of the stage's stacked tile
                        ds_b[(2 * st + 1) * TILE_NI + sw128(16 * g + k, jl)] = (uint8_t)dl[k];          // rows 64..127
                    }
                }
            };
            const bool rapido = FASE == 1 || (sh >= 1 && sh <= 30 && (FASE != 3 || (sh2 >= 1 && sh2 <= 30)));
            if (rapido) corpo(std::true_type{});
            else corpo(std::false_type{});
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
            // gq^T[digit row of k][query] += K^T chunk . (dS' digits)^T: hi digits -> columns 0..63, lo digits -> 64..127
            ok = espera(bar[B_KT + cc % NSTV], (cc / NSTV) & 1, aborta, kid, 34);
            if (ok) {
                tc_fence_depois();
                const uint64_t da = desc_sw128(sKt0 + (cc % NSTV) * TILE_A), db = desc_sw128(sbase + OFF_DS + (2 * st) * TILE_NI);
#pragma unroll
                for (int q = 0; q < 4; q++) tc_mma_i8(tmem + 2 * SB, da + 2 * q, db + 2 * q, ID_S2, (cc | q) != 0);
                tc_commit(bar[B_G + st]);
                if (cc == nvoltas - 1) tc_commit(bar[B_O]);
            }
        }
    }
    if (FASE == 1) {
        max_cta16(mgp, est + at::S_GP, red, tid);
    } else if (FASE == 2) {
        int msl = 0;
        if (tid < NI) msl = sl_s[tid] < 0 ? -sl_s[tid] : sl_s[tid];
        max_cta16(mds, est + at::S_DS, red, tid);
        if (A.limite) {
            max_cta16(mp, est + at::S_P, red, tid);
            max_cta16(mgp, est + at::S_GPQ, red, tid);
            max_cta16(msl, est + at::S_SL, red, tid);
        }
    } else {
        __syncwarp();
        ok = __all_sync(FULL, ok && espera(bar[B_O], 0, aborta, kid, 35));
        tc_fence_depois();
        int* o_s = reinterpret_cast<int*>(smem);                   // [2][128][65] over the dead operand stages
        if (ok) {
            uint32_t d1[16], d2[16];
            const int dd = 32 * (wid & 3) + lane, g = wid >> 2;
            const uint32_t t = tmem + ((uint32_t)(32 * (wid & 3)) << 16) + 2 * SB + 16 * g;
            tmem_le16(t, d1);
            tmem_le16(t + NI, d2);
#pragma unroll
            for (int k = 0; k < 16; k++) {
                o_s[dd * 65 + 16 * g + k] = (int)d1[k];
                o_s[128 * 65 + dd * 65 + 16 * g + k] = (int)d2[k];
            }
        }
        tc_fence_antes();
        __syncthreads();
        const int i = tid >> 3, d0 = (tid & 7) * 8;
        const int eds = (emg - GA) + (emv - GA) + sh - 9 + sh2, e = eds + (emk - GA);
        int o[8];
#pragma unroll
        for (int k = 0; k < 8; k++) {
            const int d = d0 + k;
            const uint32_t hhv = (uint32_t)o_s[d * 65 + i], crv = (uint32_t)o_s[(64 + d) * 65 + i] + (uint32_t)o_s[128 * 65 + d * 65 + i],
                           llv = (uint32_t)o_s[128 * 65 + (64 + d) * 65 + i];
            o[k] = junta3(hhv, crv, llv);
        }
        const size_t lin = (size_t)(linha0 + i0 + i);
        grava8(A.Gacc, A.Ge, A.Gm, A.GE, lin * 3 * D + h * HD + d0, lin * (3 * D / 32) + (h * HD + d0) / 32, o, e, kid, tid);
    }
    tc_fence_antes();
    __syncthreads();
    if (wid == 0) {
        tc_fence_depois();
        tmem_libera(tmem, 512);
    }
}
inline size_t smem_linhas_tc(int fase) { return 1024 + 4 * TILE_A + TILE_NI + TILE_Q3 + (fase == 3 ? 4 * TILE_A + 4 * TILE_NI : 0) + 640; }

// -------------------------------------------------------------------------------------------------- backward, key tiles
// gk[j] = sum_i dS'[i][j] q[i], gv[j] = sum_i P[i][j] dO[i] for the 64 keys of the tile, over the query chunks from the tile's first
// key on (everything before is causally zero).  All five operands come by TMA: q^T and dO^T digit rows (A), the tile's rows of the
// dS' digits and of P (B).  grid (ceil(T / 64), BH), 256 threads; tensor memory: three accumulators of 64 columns (256 allocated).
__global__ void __launch_bounds__(256) k_ab_colunas_tc(const __grid_constant__ CUtensorMap mQt, const __grid_constant__ CUtensorMap mGt,
                                                       const __grid_constant__ CUtensorMap mDh, const __grid_constant__ CUtensorMap mDl,
                                                       const __grid_constant__ CUtensorMap mP, const ArgsTrasTC A) {
    extern __shared__ unsigned char bruto[];
    // (pointer arithmetic on the array keeps the shared address space: a round trip through an integer makes every access generic)
    unsigned char* smem = bruto + ((1024u - (smem_u32(bruto) & 1023u)) & 1023u);
    const uint32_t sbase = smem_u32(smem);
    constexpr int NSTC = 3;                                        // a TMA load takes longer than a step: loads run two steps ahead
    constexpr uint32_t STAGE = 2 * TILE_A + 3 * TILE_NJ, OFF_BAR = NSTC * STAGE;
    const Barras bar = {sbase + OFF_BAR};                          // 0..2 full | 3..5 free | 6 o
    uint32_t* slot = reinterpret_cast<uint32_t*>(smem + OFF_BAR + 64);
    volatile int* aborta = reinterpret_cast<volatile int*>(smem + OFF_BAR + 68);
    const int T = A.T, H = A.H, D = A.D, GA = A.GA, kid = A.kid;
    const int tid = threadIdx.x, wid = tid >> 5, lane = tid & 31;
    const int ordem = blockIdx.y * gridDim.x + blockIdx.x;         // heaviest (first) key tiles of all heads first
    const int bh = ordem % gridDim.y, b = bh / H, h = bh % H, j0 = (ordem / gridDim.y) * NJ, linha0 = b * T;
    const int* est = A.est + bh * at::N_EST;
    const int nq = (T - j0 + TJ - 1) / TJ;
    auto carrega = [&](int n, int c) {                             // one thread: the five operand tiles of query chunk c, step n
        const uint32_t s = sbase + (n % NSTC) * STAGE, f = bar[n % NSTC];
        const int ic = j0 + c * TJ;
        mbar_expect_tx(f, STAGE);
        tma_2d(s, &mQt, ic, bh * 128, f);
        tma_2d(s + TILE_A, &mGt, ic, bh * 128, f);
        tma_2d(s + 2 * TILE_A, &mDh, ic, bh * T + j0, f);
        tma_2d(s + 2 * TILE_A + TILE_NJ, &mDl, ic, bh * T + j0, f);
        tma_2d(s + 2 * TILE_A + 2 * TILE_NJ, &mP, ic, bh * T + j0, f);
    };
    if (tid == 0) {
        for (int i = 0; i < 7; i++) mbar_init(bar[i], 1);
        *aborta = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    pdl_espera();                                                  // the operands are the previous kernels' outputs
    pdl_solta();
    // query chunks (128 queries from j0 + 128 c) in which stored P is zero for this key tile add nothing to gk and gv, and phase 3
    // wrote no dS' there: they are left out.  The first step (the diagonal) always stays.
    unsigned vivos = (1u << nq) - 1u;
    if (!A.limite && A.zm) {
        const unsigned m = (unsigned)A.zm[bh * ((T + NJ - 1) / NJ) + j0 / NJ];
        vivos = 1u;
        for (int c = 1; c < nq; c++)
            if (m & (3u << ((j0 + c * TJ) / NI))) vivos |= 1u << c;
    }
    const int nviv = __popc(vivos);
    auto passo = [&](int n) -> int { return (int)__fns(vivos, 0, n + 1); };      // the query chunk of live step n
    if (tid == 0)                                                  // the loads go out before anything else
        for (int n = 0; n < NSTC && n < nviv; n++) carrega(n, passo(n));
    if (wid == 0) tmem_aloca(slot, 256);
    tc_fence_antes();
    __syncthreads();
    tc_fence_depois();
    const uint32_t tmem = *slot;
    if (tid == 0) {
        bool ok = true;
        for (int c = 0; c < nviv && ok; c++) {                      // c counts the live steps
            ok = espera(bar[c % NSTC], (c / NSTC) & 1, aborta, kid, 40);
            if (!ok) break;
            tc_fence_depois();
            const uint32_t s = sbase + (c % NSTC) * STAGE;
            // the hi and lo digit tiles of dS' lie one after the other: one B operand of 128 rows -> columns 0..63 | 64..127
            const uint64_t dq = desc_sw128(s), dg = desc_sw128(s + TILE_A), dhl = desc_sw128(s + 2 * TILE_A), dp = desc_sw128(s + 2 * TILE_A + 2 * TILE_NJ);
#pragma unroll
            for (int q = 0; q < 4; q++) {
                tc_mma_i8(tmem, dq + 2 * q, dhl + 2 * q, ID_C2, (c | q) != 0);
                tc_mma_i8(tmem + 128, dg + 2 * q, dp + 2 * q, ID_CU, (c | q) != 0);
            }
            tc_commit(bar[NSTC + c % NSTC]);
            if (c >= 1 && c + 2 < nviv) {                          // step c - 1's MMAs done: its stage takes step c + 2
                ok = espera(bar[NSTC + (c - 1) % NSTC], ((c - 1) / NSTC) & 1, aborta, kid, 41);
                if (ok) carrega(c + 2, passo(c + 2));
            }
        }
        tc_commit(bar[2 * NSTC]);
    }
    __syncwarp();
    const bool ok = __all_sync(FULL, espera(bar[2 * NSTC], 0, aborta, kid, 42));
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
        for (int t = tid; t < NJ * 8; t += 256) {
            const int jl = t >> 3, d0 = (t & 7) * 8, j = min(j0 + jl, T - 1);      // rows beyond T (whole groups of 8 lanes) compute and store nothing
            const bool grava = j0 + jl < T;
            int gk[8], gv[8];
#pragma unroll
            for (int k = 0; k < 8; k++) {
                const int d = d0 + k;
                const uint32_t hhv = (uint32_t)o_s[d * 65 + jl], crv = (uint32_t)o_s[(64 + d) * 65 + jl] + (uint32_t)o_s[(128 + d) * 65 + jl],
                               llv = (uint32_t)o_s[(128 + 64 + d) * 65 + jl];
                gk[k] = junta3(hhv, crv, llv);
                gv[k] = (int)(((uint32_t)o_s[(256 + d) * 65 + jl] << 7) + (uint32_t)o_s[(256 + 64 + d) * 65 + jl]);
            }
            const size_t lin = (size_t)(linha0 + j), p = lin * 3 * D + D + h * HD + d0, pe = lin * (3 * D / 32) + (D + h * HD + d0) / 32;
            grava8(A.Gacc, A.Ge, A.Gm, A.GE, p, pe, gk, e_k, kid, t, grava);
            grava8(A.Gacc, A.Ge, A.Gm, A.GE, p + D, pe + D / 32, gv, e_v, kid, t, grava);
        }
    }
    if (wid == 0) {
        tc_fence_depois();
        tmem_libera(tmem, 256);
    }
}
inline size_t smem_colunas_tc() { return 1024 + 3 * (2 * TILE_A + 3 * TILE_NJ) + 128; }

}  // namespace atc

// -------------------------------------------------------------------------------------------------- host side
static size_t atc_arredonda(size_t x) { return (x + 1023) & ~(size_t)1023; }

// head dimension 64, whole row tiles of 64 queries and at least one full key chunk (the TMA boxes are 128 tokens wide)
static bool atc_serve(int blk, int T, int H, int D) { return D == H * atc::HD && T % atc::NI == 0 && T >= 128 && T <= 1024 && D % blk == 0 && (blk == 32 || blk == 128); }

// forward: preparation (q, k row layout; v transposed) + the tensor-core kernel
// Qm / QE: block output (jt_quant of the raw output) instead of Oacc / Oe, block length 32 only; nullptr = raw output
static int atencao_frente_tc(int blk, const int8_t* qm, const int8_t* qE, int* Oacc, int16_t* Oe, int8_t* Qm, int8_t* QE, uint8_t* P, int Bt, int T, int H,
                             int D, int GA, int kid, cudaStream_t st) {
    if (Qm && (blk != 32 || !QE)) return (int)cudaErrorInvalidValue;
    const int BH = Bt * H;
    // head-maximum exponents [BH][4], then the largest squared row norms of q and k per 128 tokens [BH][2][ceil(T/128)]
    const size_t b_em = atc_arredonda((size_t)BH * 16 + (size_t)BH * 2 * ((T + 127) / 128) * 4), b_lin = atc_arredonda((size_t)BH * T * 128);
    unsigned char* ws = nullptr;
    if (int r = at_ws(b_em + 3 * b_lin, st, reinterpret_cast<void**>(&ws))) return r;
    int* em = reinterpret_cast<int*>(ws);
    int8_t *Q2 = reinterpret_cast<int8_t*>(ws + b_em), *K2 = Q2 + b_lin, *Vt2 = K2 + b_lin;
    atc::ArgsPrep Pp = {qm, qE, nullptr, nullptr, {Q2, K2, nullptr, nullptr}, {nullptr, nullptr, Vt2, nullptr}, em, nullptr, T > 2 * atc::TJ ? em + 4 * BH : nullptr, T, H, D, GA, blk};
    lanca_pdl(atc::k_at_prep, dim3(dim3((T + 127) / 128, BH, 3)), dim3(256), 0, st, Pp);
    CUtensorMap mQ, mK, mVt;
    if (!(faz_mapa(&mQ, Q2, BH * T, 128, atc::NI) && faz_mapa(&mK, K2, BH * T, 128, 128) && faz_mapa(&mVt, Vt2, BH * 128, T, 128)))
        return (int)cudaErrorInvalidValue;
    const size_t sm = atc::smem_frente_tc(T);
    cudaError_t c = at_smem(atc::k_atencao_tc, sm);
    if (c != cudaSuccess) return (int)c;
    lanca_pdl(atc::k_atencao_tc, dim3(dim3(T / atc::NI, BH)), dim3(atc::NTL), sm, st, mQ, mK, mVt, em, Oacc, Oe, Qm, QE, P, T, H, D, GA, kid);
    return (int)cudaGetLastError();
}

// backward: preparation (v, dO row layout; q, k, dO transposed), the three row-tile phases, the key-tile kernel
static int atencao_tras_tc(int blk, const int8_t* gom, const int8_t* goE, const int8_t* qm, const int8_t* qE, const uint8_t* P, int* Gacc, int16_t* Ge,
                           int8_t* Gm, int8_t* GE, int Bt, int T, int H, int D, int GA, int limite, int kid, cudaStream_t st) {
    if (Gm && (blk != 32 || !GE)) return (int)cudaErrorInvalidValue;
    const int BH = Bt * H;
    const size_t b_est = atc_arredonda((size_t)BH * (at::N_EST + T + 4 + 16) * sizeof(int)), b_lin = atc_arredonda((size_t)BH * T * 128),
                 b_ds = atc_arredonda((size_t)BH * T * T);
    unsigned char* ws = nullptr;
    if (int r = at_ws(b_est + 5 * b_lin + 2 * b_ds, st, reinterpret_cast<void**>(&ws))) return r;
    int* est = reinterpret_cast<int*>(ws);
    int* sl = est + (size_t)BH * at::N_EST;
    int* em = sl + (size_t)BH * T;
    int* zm = em + (size_t)BH * 4;                               // [BH][ceil(T/64)] (T <= 1024: at most 16 per head)
    int8_t *V2 = reinterpret_cast<int8_t*>(ws + b_est), *G2 = V2 + b_lin, *Qt2 = G2 + b_lin, *Kt2 = Qt2 + b_lin, *Gt2 = Kt2 + b_lin;
    int8_t *DSh = Gt2 + b_lin, *DSl = DSh + b_ds;
    cudaError_t c;
    atc::ArgsPrep Pp = {qm, qE, gom, goE, {nullptr, nullptr, V2, G2}, {Qt2, Kt2, nullptr, Gt2}, em, est, nullptr, T, H, D, GA, blk};
    lanca_pdl(atc::k_at_prep, dim3(dim3((T + 127) / 128, BH, 4)), dim3(256), 0, st, Pp);
    CUtensorMap mV, mG, mKt, mQt, mGt, mDh, mDl, mP;
    if (!(faz_mapa(&mV, V2, BH * T, 128, 128) && faz_mapa(&mG, G2, BH * T, 128, atc::NI) && faz_mapa(&mKt, Kt2, BH * 128, T, 128) &&
          faz_mapa(&mQt, Qt2, BH * 128, T, 128) && faz_mapa(&mGt, Gt2, BH * 128, T, 128) && faz_mapa(&mDh, DSh, BH * T, T, atc::NJ) &&
          faz_mapa(&mDl, DSl, BH * T, T, atc::NJ) && faz_mapa(&mP, P, BH * T, T, atc::NJ)))
        return (int)cudaErrorInvalidValue;
    // the map of zero tiles of P pays from three key chunks on (T > 256): below that nearly every chunk is next to the diagonal
    const bool com_mapa = !limite && T > 256;
    atc::ArgsTrasTC A = {P, Gacc, Ge, est, sl, em, com_mapa ? zm : nullptr, DSh, DSl, Gm, GE, T, H, D, GA, limite, kid};
    if (com_mapa) lanca_pdl(atc::k_p_mapa, dim3((T + atc::NJ - 1) / atc::NJ, BH), dim3(256), 0, st, P, zm, T);
    const dim3 grade(T / atc::NI, BH);
    if (limite) {
        at::ArgsTras L = {gom, goE, qm, qE, P, Gacc, Ge, est, sl, nullptr, T, H, D, GA, blk, limite, kid};
        at::k_lim<atc::HD><<<BH, 256, 0, st>>>(L);
    } else {
        if ((c = at_smem(atc::k_ab_linhas_tc<1>, atc::smem_linhas_tc(1))) != cudaSuccess) return (int)c;
        lanca_pdl(atc::k_ab_linhas_tc<1>, dim3(grade), dim3(atc::NTL), atc::smem_linhas_tc(1), st, mV, mG, mKt, A);
    }
    if ((c = at_smem(atc::k_ab_linhas_tc<2>, atc::smem_linhas_tc(2))) != cudaSuccess) return (int)c;
    lanca_pdl(atc::k_ab_linhas_tc<2>, dim3(grade), dim3(atc::NTL), atc::smem_linhas_tc(2), st, mV, mG, mKt, A);
    if ((c = at_smem(atc::k_ab_linhas_tc<3>, atc::smem_linhas_tc(3))) != cudaSuccess) return (int)c;
    lanca_pdl(atc::k_ab_linhas_tc<3>, dim3(grade), dim3(atc::NTL), atc::smem_linhas_tc(3), st, mV, mG, mKt, A);
    if ((c = at_smem(atc::k_ab_colunas_tc, atc::smem_colunas_tc())) != cudaSuccess) return (int)c;
    lanca_pdl(atc::k_ab_colunas_tc, dim3(dim3((T + atc::NJ - 1) / atc::NJ, BH)), dim3(256), atc::smem_colunas_tc(), st, mQt, mGt, mDh, mDl, mP, A);
    return (int)cudaGetLastError();
}

}  // namespace jt
