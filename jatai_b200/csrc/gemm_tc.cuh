// Tensor-core block GEMM for sm_100a: tcgen05.mma kind::i8 with the accumulator in tensor memory, operands
// staged by TMA, and the per-K-block alignment / rounding of the reference specification done on the CUDA
// cores between the tensor memory and the register accumulators.
//
//   C[M,N] = A[M,K] . B[N,K]^T, operands blocked along K (jatai_cuda/ops.py:95-108):
//   acc_ij = sum over K-blocks b of rnd(p_ijb << 4, (RA_i - ea_ib) + (RB_j - eb_jb)),  p = exact int8 dot product.
//
// The rounding of every block's partial product depends on its value, so partial products of different
// blocks can not be summed by the tensor core.  One MMA instruction of kind::i8 has K = 32: with BLK = 32 every
// instruction starts a fresh accumulator (tensor-memory stage) that is drained, aligned and added in registers;
// with BLK = 128 four instructions accumulate in tensor memory before one drain.
//
// CTA = one 128 x TNv tile of C (optionally one K range of it: split-K for raw outputs), 2 + TNv / 8 warps (TNv = 128 below):
//   warp 0       TMA producer (one lane): A and B tiles of 128 rows x 128 bytes of K, SWIZZLE_128B, NST-stage ring;
//                all 32 lanes also build, ahead of the drain, the table of column scales 2^-(RB_j - eb_jb) it reads
//   warp 1       allocates tensor memory, issues the MMAs (one thread), frees tensor memory
//   warps 2..17  drain: thread = one row of the tile (tcgen05.ld 32x32b), 32 columns each (4 warps per scheduler hide
//                the tensor-memory load latency), then the output stage
// Every wait on an mbarrier is bounded: on a timeout the CTA records E_TEMPO, raises an abort flag that turns all
// later waits into no-ops, and leaves through the normal exit (tensor memory is freed).
#pragma once
#include <cuda.h>
#include "gemm_comum.cuh"

namespace jt {
namespace tc {

constexpr int TM = 128, KC = 128, NST = 4, NTM = 4, NTB = 4;
constexpr uint32_t A_BYTES = TM * KC;
// everything that depends on the tile width TNv (columns of C per CTA): 128, or 64 for shapes whose 128-wide tiling
// would leave most SMs without a CTA (block 32 only: a 128-column exponent block does not fit a 64-column tile)
template <int TNv, int VIA>
struct Cfg {
    static constexpr int N_DW = TNv / 8;                       // drain warps: 4 lane quarters x (TNv / 32) column groups
    static constexpr int N_EPI = N_DW * 32, N_THR = 64 + N_EPI, PITCHv = TNv + 4;
    static constexpr uint32_t B_BYTES = TNv * KC, STAGE_BYTES = A_BYTES + B_BYTES;
    // the staged accumulators of the output stage reuse the operand ring: when a drain thread stores its accumulators
    // it has seen the commit of the last MMA, so every TMA load has landed and every operand read has finished
    static constexpr uint32_t OFF_ACC = 0;
    static_assert(TM * PITCHv * 4 <= NST * STAGE_BYTES, "staged accumulators must fit in the operand ring");
    static constexpr uint32_t OFF_TAB = NST * STAGE_BYTES;                  // scale table ring: [NTB][4][TNv] floats
    static constexpr uint32_t OFF_RA = OFF_TAB + NTB * 4 * TNv * 4;
    static constexpr uint32_t OFF_RB = OFF_RA + TM * 4;
    static constexpr uint32_t OFF_RBF = OFF_RB + TNv * 4;                   // 2^(RB_j - minimum of j's block), floats
    static constexpr uint32_t OFF_RBM = OFF_RBF + TNv * 4;                  // minimum and maximum RB of each block: int[4] + int[4]
    static constexpr uint32_t OFF_BAR = OFF_RBM + 32;
    static constexpr uint32_t OFF_MISC = OFF_BAR + (2 * NST + 2 * NTM + 2 * NTB) * 8;
    static constexpr uint32_t OFF_C127 = (OFF_MISC + 16 + 1023) / 1024 * 1024;   // 1 KB of the byte 127: the constant operand
    static constexpr uint32_t SMEM_BYTES = OFF_C127 + 1024 + 1024;          // + slack to align the base to 1024 bytes
    // 64-column tiles: two CTAs per SM (2 x 256 columns of tensor memory, 2 x ~100 KB of shared memory, <= 102 registers):
    // the prologue and the output stage of one overlap the main loop of the other
    static constexpr int CTAS_SM = TNv == 64 ? 2 : 1;
    // instruction descriptor kind::i8: D = s32, A = B = s8, both K-major, N = TNv, M = 128
    static constexpr uint32_t IDESC = (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(TNv >> 3) << 17) | ((uint32_t)(TM >> 4) << 24);
};
constexpr long long LIMITE_CICLOS = 4000000000LL;              // ~2 s at B200 clocks
__device__ long long g_limite_espera = LIMITE_CICLOS;          // the limit in force (jt_espera_limite); read on the slow path of a wait only
__device__ int g_sem_cargas = 0;                               // test switch (jt_gemm_sem_cargas): the producer issues no operand load, so the
                                                               // first wait of the MMA warp runs out with nothing asynchronous in flight
constexpr uint32_t MAGIA = 0x4B400000u;                        // bit pattern of 1.5 * 2^23
constexpr float MAGIA_F = 12582912.0f;
constexpr int DESLOC = 32 * 127 * 127;                         // the largest |partial product| of 32 int8 pairs

// ------------------------------------------------------------------------------------------ PTX wrappers
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t n) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(n) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t par) {
    uint32_t ok;
    asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
                 : "=r"(ok) : "r"(bar), "r"(par) : "memory");
    return ok != 0;
}
// bounded wait; false = gave up (abort flag raised by this or another thread)
__device__ __forceinline__ bool espera(uint32_t bar, uint32_t par, volatile int* aborta, int kid, int onde) {
    long long t0 = 0;
    for (int it = 1;; it++) {
        if (mbar_try(bar, par)) return true;
        if (*aborta) return false;
        if ((it & 255) == 0) {
            const long long agora = clock64();
            if (t0 == 0) t0 = agora;
            else if (*reinterpret_cast<volatile int*>(&g_erro.codigo) == E_TEMPO && *reinterpret_cast<volatile int*>(&g_erro.n) != 0) {
                *aborta = 1;                     // a wait has already expired somewhere in this step: do not wait out another limit
                return false;
            } else if (agora - t0 > *reinterpret_cast<volatile long long*>(&g_limite_espera)) {
                *aborta = 1;
                reporta(E_TEMPO, kid, onde, par, blockIdx.x + 65536LL * blockIdx.y);
                return false;
            }
        }
    }
}
// The bounded wait on its own: one warp waits for a phase of an mbarrier that nothing ever completes, gives up when the limit
// in force has passed, records E_TEMPO (place 99) and leaves normally.  No copy, MMA or other CTA is involved.
__global__ void k_teste_espera(int kid, int* saiu) {
    __shared__ __align__(8) unsigned long long barra;
    __shared__ int aborta_s;
    if (threadIdx.x == 0) {
        mbar_init(smem_u32(&barra), 1);
        aborta_s = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    const bool ok = espera(smem_u32(&barra), 0, &aborta_s, kid, 99);
    if (threadIdx.x == 0) *saiu = ok ? 1 : 2;                     // 2 = gave up, as it must
}
__device__ __forceinline__ void tma_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar) : "memory");
}
__device__ __forceinline__ void tc_fence_antes() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_depois() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_mma_i8(uint32_t d_tmem, uint64_t da, uint64_t db, uint32_t idesc, uint32_t acumula) {
    asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
                 " tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n}"
                 ::"r"(d_tmem), "l"(da), "l"(db), "r"(idesc), "r"(acumula) : "memory");
}
// shared-memory matrix descriptor: K-major operand, 128-byte swizzle, 8-row groups 1024 bytes apart
__device__ __forceinline__ uint64_t desc_sw128(uint32_t addr) {
    return (uint64_t)((addr >> 4) & 0x3FFF) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) | ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}

#define JT_O4(a, i) "=r"(a[i]), "=r"(a[i + 1]), "=r"(a[i + 2]), "=r"(a[i + 3])
#define JT_O16(a, i) JT_O4(a, i), JT_O4(a, i + 4), JT_O4(a, i + 8), JT_O4(a, i + 12)
#define JT_O32(a, i) JT_O16(a, i), JT_O16(a, i + 16)
// 32 consecutive columns of this thread's tensor-memory lane -> registers; returns when the data has arrived
__device__ __forceinline__ void tmem_le32(uint32_t taddr, uint32_t (&d)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,"
        "%24,%25,%26,%27,%28,%29,%30,%31}, [%32];\n"
        "tcgen05.wait::ld.sync.aligned;\n"
        : JT_O32(d, 0)
        : "r"(taddr)
        : "memory");
}

// 16 consecutive columns of this thread's lane from each of two tensor-memory addresses (two K slices); one wait for both
__device__ __forceinline__ void tmem_le16x2(uint32_t ta, uint32_t tb, uint32_t (&a)[16], uint32_t (&b)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%32];\n"
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%33];\n"
        "tcgen05.wait::ld.sync.aligned;\n"
        : JT_O16(a, 0), JT_O16(b, 0)
        : "r"(ta), "r"(tb)
        : "memory");
}
__device__ __forceinline__ void tmem_le8x2(uint32_t ta, uint32_t tb, uint32_t (&a)[8], uint32_t (&b)[8]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%16];\n"
        "tcgen05.ld.sync.aligned.32x32b.x8.b32 {%8,%9,%10,%11,%12,%13,%14,%15}, [%17];\n"
        "tcgen05.wait::ld.sync.aligned;\n"
        : JT_O4(a, 0), JT_O4(a, 4), JT_O4(b, 0), JT_O4(b, 4)
        : "r"(ta), "r"(tb)
        : "memory");
}
// two fp32 lanes per instruction (fma.rn.f32x2): the align/round loop is bound by instruction issue, not by the FMA pipe
__device__ __forceinline__ uint64_t par(uint32_t lo, uint32_t hi) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "r"(lo), "r"(hi));
    return r;
}
__device__ __forceinline__ uint64_t par_f(float lo, float hi) { return par(__float_as_uint(lo), __float_as_uint(hi)); }
__device__ __forceinline__ void separa(uint64_t v, uint32_t& lo, uint32_t& hi) { asm("mov.b64 {%0, %1}, %2;" : "=r"(lo), "=r"(hi) : "l"(v)); }
__device__ __forceinline__ uint64_t ffma2(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}

__device__ __forceinline__ float pot2(int e) { return __int_as_float((127 + e) << 23); }      // 2^e, -126 <= e <= 127

// How a K-block's partial product p (exact int32 from tensor memory, |p| <= 32 * 127^2 < 2^19) becomes rnd(p << 4, sa + sb):
// VIA 1 (block 32): every slice gets a second MMA of two constant operands (all bytes 127) onto the same accumulator, so what
//        the drain reads is p' = p + 32*127^2 >= 0.  Read as a float, the bit pattern of a non-negative integer below 2^23 is the
//        subnormal p' * 2^-149 - an exact int -> float conversion that costs no instruction.  One FMA scales it by 2^(123-sa) and
//        takes the constant off (exact: the result is (p' - 32*127^2) * 2^(-26-sa)), a second FMA against 1.5*2^23 scales by
//        2^(30-sb) and rounds half to even in its single rounding; the result's bit pattern is added to the accumulator (the
//        pattern of 1.5*2^23 times the slice count comes off at the end).  Two slices are drained together so that one three-input
//        add serves both, and the FMAs are the packed two-lane form.  The rounding is exact while |p * 2^(4-s)| < 2^22, i.e.
//        always except s = 0 with |p| >= 2^18, and exactly then the sum leaves [2^23, 2^24]: its exponent field changes.  The bit
//        patterns of a half chunk's results are OR-ed as they are added, and a warp in which some pattern's top nine bits are not
//        those of 1.5*2^23 reads the half chunk again (the stages are handed back only after this vote), takes the fast results
//        off and adds VIA 2's conversions instead.
// VIA 2: exact float product, cvt.rni to int (valid for every input; block 128, where four MMAs accumulate before a drain).
template <int BLK, int MODO, int VIA, int TNv>
__global__ void __launch_bounds__(Cfg<TNv, VIA>::N_THR, Cfg<TNv, VIA>::CTAS_SM) k_gemm_tc(const __grid_constant__ CUtensorMap mapA, const __grid_constant__ CUtensorMap mapB,
                                                      const int8_t* __restrict__ EA, const int8_t* __restrict__ EB,
                                                      const int8_t* __restrict__ RAg, const int8_t* __restrict__ RBg, SaidaGemm S, int M, int N,
                                                      int K, int pedacos_por_parte, int kid) {
    constexpr int NQ = KC / BLK;                 // K-blocks per 128-byte chunk: 4 (BLK 32) or 1 (BLK 128)
    using C_ = Cfg<TNv, VIA>;
    constexpr int N_DW = C_::N_DW, N_EPI = C_::N_EPI, PITCHv = C_::PITCHv;
    constexpr bool PARES = BLK == 32 && VIA == 1;
    static_assert(VIA != 1 || BLK == 32, "the FMA rounding is written for one MMA per drain");
    constexpr uint32_t STAGE_BYTES = C_::STAGE_BYTES, OFF_ACC = C_::OFF_ACC, OFF_TAB = C_::OFF_TAB, OFF_RA = C_::OFF_RA, OFF_RB = C_::OFF_RB, OFF_RBF = C_::OFF_RBF, OFF_RBM = C_::OFF_RBM,
                       OFF_BAR = C_::OFF_BAR, OFF_MISC = C_::OFF_MISC, IDESC = C_::IDESC;
    static_assert(TNv == 128 || (TNv == 64 && BLK == 32), "64-column tiles exist for block 32 only");
    extern __shared__ unsigned char smem_bruto[];
    // (pointer arithmetic on the array keeps the shared address space: a round trip through an integer makes every access generic)
    unsigned char* smem = smem_bruto + ((1024u - (smem_u32(smem_bruto) & 1023u)) & 1023u);
    const uint32_t sbase = smem_u32(smem);
    int* acc_s = reinterpret_cast<int*>(smem + OFF_ACC);
    float* tabB = reinterpret_cast<float*>(smem + OFF_TAB);          // [NTB][4][TN]
    int* RAs = reinterpret_cast<int*>(smem + OFF_RA);
    int* RBs = reinterpret_cast<int*>(smem + OFF_RB);
    float* RBf = reinterpret_cast<float*>(smem + OFF_RBF);
    int* RBm = reinterpret_cast<int*>(smem + OFF_RBM);
    const uint32_t bar_full = sbase + OFF_BAR, bar_empty = bar_full + NST * 8, bar_tfull = bar_empty + NST * 8, bar_tempty = bar_tfull + NTM * 8;
    const uint32_t bar_bfull = bar_tempty + NTM * 8, bar_bempty = bar_bfull + NTB * 8;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + OFF_MISC);
    volatile int* aborta = reinterpret_cast<volatile int*>(smem + OFF_MISC + 4);

    const int tid = threadIdx.x, wid = tid >> 5, lane = tid & 31;
    const int m0 = blockIdx.y * TM, n0 = blockIdx.x * TNv;
    const int nb = K / BLK;
    const int ped0 = blockIdx.z * pedacos_por_parte;             // first 128-byte chunk of this CTA's K range
    const int nfatias = pedacos_por_parte * NQ;                  // drains (K-blocks) this CTA performs

    if (tid == 0) {
        for (int i = 0; i < NST; i++) { mbar_init(bar_full + 8 * i, 1); mbar_init(bar_empty + 8 * i, 1); }
        for (int i = 0; i < NTM; i++) { mbar_init(bar_tfull + 8 * i, 1); mbar_init(bar_tempty + 8 * i, N_DW); }
        for (int i = 0; i < NTB; i++) { mbar_init(bar_bfull + 8 * i, 32); mbar_init(bar_bempty + 8 * i, N_DW); }
        *aborta = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (PARES) {
        if (tid < 64) reinterpret_cast<uint4*>(smem + C_::OFF_C127)[tid] = make_uint4(0x7F7F7F7Fu, 0x7F7F7F7Fu, 0x7F7F7F7Fu, 0x7F7F7F7Fu);
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");          // the MMA reads it through the async proxy
    }
    if (tid < TM) RAs[tid] = -128;
    if (tid < TNv) RBs[tid] = -128;
    if (tid < 8) RBm[tid] = tid < 4 ? 1000 : -1000;
    if (wid == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(NTM * TNv) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_antes();
    __syncthreads();
    tc_fence_depois();
    const uint32_t tmem = *tmem_slot;
    pdl_espera();                                  // everything above touches no global memory: it overlaps the predecessor's tail
    pdl_solta();

    if (wid == 0) {
        // ------------------------------------------------------------------ TMA producer + column scale tables
        // lane l owns columns l, l+32, ... of the tile: their row maxima RB and, per chunk, their scales
        constexpr int NC = TNv / 32;
        auto carrega = [&](int i) {
            const int s = i % NST;
            mbar_expect_tx(bar_full + 8 * s, STAGE_BYTES);
            tma_2d(sbase + s * STAGE_BYTES, &mapA, (ped0 + i) * KC, m0, bar_full + 8 * s);
            tma_2d(sbase + s * STAGE_BYTES + A_BYTES, &mapB, (ped0 + i) * KC, n0, bar_full + 8 * s);
        };
        // the first NST stages are free: their loads start before anything else, the row maxima (computed by the
        // drain threads meanwhile) are only needed for the scale tables
        const bool sem_cargas = *reinterpret_cast<volatile int*>(&g_sem_cargas) != 0;
        if (lane == 0 && !sem_cargas)
            for (int i = 0; i < NST && i < pedacos_por_parte; i++) carrega(i);
        const int8_t* ebc[NC];
        uint32_t w[NC];                           // block exponents of this lane's columns for the next chunk, read one chunk ahead
        auto le_w = [&](int i) {
#pragma unroll
            for (int k = 0; k < NC; k++)
                w[k] = NQ == 4 ? *reinterpret_cast<const uint32_t*>(ebc[k] + 4 * i) : (uint32_t)(uint8_t)ebc[k][i];
        };
#pragma unroll
        for (int k = 0; k < NC; k++) ebc[k] = EB + (size_t)(n0 + lane + 32 * k) * nb + (size_t)ped0 * NQ;
        le_w(0);
        __syncwarp();
        asm volatile("bar.sync 2, %0;" ::"n"(N_EPI + 32) : "memory");
        int RBc[NC];
#pragma unroll
        for (int k = 0; k < NC; k++) RBc[k] = RBs[lane + 32 * k];
        bool ok = true;
        for (int i = 0; i < pedacos_por_parte; i++) {
            if (lane == 0 && i >= NST) {
                ok = espera(bar_empty + 8 * (i % NST), ((i / NST) & 1) ^ 1, aborta, kid, 1);
                if (ok && !sem_cargas) carrega(i);
            }
            ok = __all_sync(FULL, ok);
            if (!ok) break;
            const int sl = i % NTB;
            ok = __all_sync(FULL, espera(bar_bempty + 8 * sl, ((i / NTB) & 1) ^ 1, aborta, kid, 5));
            if (!ok) break;
#pragma unroll
            for (int k = 0; k < NC; k++)
#pragma unroll
                for (int q = 0; q < NQ; q++) {
                    const int sb = min(RBc[k] - (int)(int8_t)(w[k] >> (8 * q)), 40);
                    tabB[(sl * 4 + q) * TNv + lane + 32 * k] = pot2((PARES ? 30 : 0) - sb);
                }
            mbar_arrive(bar_bfull + 8 * sl);
            if (i + 1 < pedacos_por_parte) le_w(i + 1);
        }
    } else if (wid == 1) {
        // ------------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            int f = 0;
            bool ok = true;
            const uint64_t d127 = desc_sw128(sbase + C_::OFF_C127) & ~((uint64_t)0x3FFF << 32);
            for (int i = 0; i < pedacos_por_parte && ok; i++) {
                const int s = i % NST;
                if (!espera(bar_full + 8 * s, (i / NST) & 1, aborta, kid, 2)) break;
                tc_fence_depois();
                const uint64_t da = desc_sw128(sbase + s * STAGE_BYTES), db = desc_sw128(sbase + s * STAGE_BYTES + A_BYTES);
                if (BLK == 32 && VIA == 1) {
                    // two slices per hand-over (the drain takes them together): barriers of the even stages only.  The constant
                    // product 32 * 127 * 127 goes in first (every 8-row group of both operands is the same 1 KB of the byte 127:
                    // group stride 0), the slices' products on top of it.
#pragma unroll
                    for (int q = 0; q < 4; q += 2, f += 2) {
                        const int t = f % NTM;
                        if (!espera(bar_tempty + 8 * t, ((f / NTM) & 1) ^ 1, aborta, kid, 3)) { ok = false; break; }
                        tc_fence_depois();
                        tc_mma_i8(tmem + t * TNv, d127, d127, IDESC, 0);
                        tc_mma_i8(tmem + (t + 1) * TNv, d127, d127, IDESC, 0);
                        tc_mma_i8(tmem + t * TNv, da + 2 * q, db + 2 * q, IDESC, 1);               // +32 bytes of K per instruction
                        tc_mma_i8(tmem + (t + 1) * TNv, da + 2 * q + 2, db + 2 * q + 2, IDESC, 1);
                        tc_commit(bar_tfull + 8 * t);
                    }
                } else if (BLK == 32) {
#pragma unroll
                    for (int q = 0; q < 4; q++, f++) {
                        const int t = f % NTM;
                        if (!espera(bar_tempty + 8 * t, ((f / NTM) & 1) ^ 1, aborta, kid, 3)) { ok = false; break; }
                        tc_fence_depois();
                        tc_mma_i8(tmem + t * TNv, da + 2 * q, db + 2 * q, IDESC, 0);               // +32 bytes of K per instruction
                        tc_commit(bar_tfull + 8 * t);
                    }
                } else {
                    const int t = f % NTM;
                    if (!espera(bar_tempty + 8 * t, ((f / NTM) & 1) ^ 1, aborta, kid, 3)) break;
                    tc_fence_depois();
#pragma unroll
                    for (int q = 0; q < 4; q++) tc_mma_i8(tmem + t * TNv, da + 2 * q, db + 2 * q, IDESC, q > 0);
                    tc_commit(bar_tfull + 8 * t);
                    f++;
                }
                tc_commit(bar_empty + 8 * s);
            }
        }
    } else {
        // ------------------------------------------------------------------ drain + output stage
        const int et = tid - 64;                                  // 0..511
        const int quarto = wid & 3;                               // tensor-memory lanes this warp may read
        const int cg = (wid - 2) >> 2;                            // column group of 32 within the tile
        const int lin = quarto * 32 + lane;                       // row of the tile = tensor-memory lane
        const int8_t* ea_lin = EA + (size_t)(m0 + lin) * nb + (size_t)ped0 * NQ;
        auto le_exp = [&](int c) -> uint32_t {
            if (NQ == 4) return *reinterpret_cast<const uint32_t*>(ea_lin + 4 * c);
            return (uint32_t)(uint8_t)ea_lin[c];
        };
        uint32_t eaw = le_exp(0), eaw_prox = 0;
        // row maxima of the tile's 128 rows of A and TNv rows of B: all drain threads share the reads (16-byte pieces,
        // one round trip to L2) and combine in shared memory
        {
            const bool pecas = (nb & 15) == 0;
            const int ppl = pecas ? nb >> 4 : 1, npec = (TM + TNv) * ppl;
            for (int idx = et; idx < npec; idx += N_EPI) {
                const int l = idx / ppl, pc = idx - l * ppl;
                const bool deA = l < TM;
                const int8_t* Rg = deA ? RAg : RBg;
                const int lg = deA ? m0 + l : n0 + l - TM;
                int v;
                if (Rg) {
                    if (pc) continue;
                    v = Rg[lg];
                } else {
                    const int8_t* pe = (deA ? EA : EB) + (size_t)lg * nb;
                    v = pecas ? max_expoentes(pe + 16 * pc, 16) : max_expoentes(pe, nb);
                }
                atomicMax(deA ? &RAs[l] : &RBs[l - TM], v);
            }
        }
        asm volatile("bar.sync 2, %0;" ::"n"(N_EPI + 32) : "memory");
        const int RA = RAs[lin];
        if (MODO != 1 && et < TNv) {
            // what the fp32 path of the output stage needs: each block's extreme column exponents and the column scales
            const int rb = RBs[et], b = et / BLK;
            int mn = rb, mx = rb;
#pragma unroll
            for (int o = 16; o; o >>= 1) { mn = min(mn, __shfl_xor_sync(FULL, mn, o)); mx = max(mx, __shfl_xor_sync(FULL, mx, o)); }
            if (BLK > 32) {
                if (lane == 0) { atomicMin(&RBm[b], mn); atomicMax(&RBm[4 + b], mx); }
                asm volatile("bar.sync 3, %0;" ::"n"(TNv) : "memory");
                mn = RBm[b];
            } else if (lane == 0) { RBm[b] = mn; RBm[4 + b] = mx; }
            RBf[et] = pot2(min(rb - mn, 100));
        }
        int acc[32];
#pragma unroll
        for (int j = 0; j < 32; j++) acc[j] = 0;
        int f = 0;
        bool ok = true;
        if constexpr (PARES) {
            static_assert(NQ == NTM, "one tensor-memory stage per K-block of a chunk");
            const uint64_t magia2 = par_f(MAGIA_F, MAGIA_F);
            for (int c = 0; c < pedacos_por_parte && ok; c++) {
                const int sl = c % NTB;
                if (c + 1 < pedacos_por_parte) eaw_prox = le_exp(c + 1);
                ok = __all_sync(FULL, espera(bar_bfull + 8 * sl, (c / NTB) & 1, aborta, kid, 6));
                if (!ok) break;
#pragma unroll
                for (int h = 0; h < 2; h++) {
                    const int t0 = 2 * h, t1 = 2 * h + 1;
                    ok = __all_sync(FULL, espera(bar_tfull + 8 * t0, c & 1, aborta, kid, 4));      // one hand-over for both stages
                    if (!ok) break;
                    tc_fence_depois();
                    const int sa0 = min(RA - (int)(int8_t)(eaw >> (16 * h)), 40), sa1 = min(RA - (int)(int8_t)(eaw >> (16 * h + 8)), 40);
                    const uint32_t base_h = tmem + ((uint32_t)(quarto * 32) << 16) + cg * 32;
                    const float* tb_h = tabB + (sl * 4 + t0) * TNv + cg * 32;
                    const float fa0 = pot2(123 - sa0), fa1 = pot2(123 - sa1);
                    const float cn0 = -(float)DESLOC * pot2(GG - 30 - sa0), cn1 = -(float)DESLOC * pot2(GG - 30 - sa1);
                    const uint64_t fa0p = par_f(fa0, fa0), fa1p = par_f(fa1, fa1), cn0p = par_f(cn0, cn0), cn1p = par_f(cn1, cn1);
                    uint32_t ou = 0;
#pragma unroll
                    for (int hf = 0; hf < 4; hf++) {                   // 8 columns of two slices at a time
                        uint32_t d0[8], d1[8];                         // p' = p + 32*127^2: as floats, the subnormals p' * 2^-149
                        tmem_le8x2(base_h + hf * 8 + t0 * TNv, base_h + hf * 8 + t1 * TNv, d0, d1);
                        const float* tb0 = tb_h + hf * 8;
                        const float* tb1 = tb0 + TNv;
#pragma unroll
                        for (int k4 = 0; k4 < 2; k4++) {
                            const ulonglong2 b0 = reinterpret_cast<const ulonglong2*>(tb0)[k4], b1 = reinterpret_cast<const ulonglong2*>(tb1)[k4];
                            const uint64_t fb0[2] = {b0.x, b0.y}, fb1[2] = {b1.x, b1.y};
#pragma unroll
                            for (int k2 = 0; k2 < 2; k2++) {
                                const int k = 4 * k4 + 2 * k2;
                                const uint64_t r0 = ffma2(ffma2(par(d0[k], d0[k + 1]), fa0p, cn0p), fb0[k2], magia2);
                                const uint64_t r1 = ffma2(ffma2(par(d1[k], d1[k + 1]), fa1p, cn1p), fb1[k2], magia2);
                                uint32_t x0, y0, x1, y1;
                                separa(r0, x0, y0);
                                separa(r1, x1, y1);
                                ou |= x0 | y0;
                                ou |= x1 | y1;
                                acc[hf * 8 + k] += (int)(x0 + x1);
                                acc[hf * 8 + k + 1] += (int)(y0 + y1);
                            }
                        }
                    }
                    if (__any_sync(FULL, (ou & 0xFF800000u) != (MAGIA & 0xFF800000u))) {
                        // some result left the window of the rounding constant: take the fast results off again, add the conversions
                        const float ga0 = pot2(GG - 30 - sa0), ga1 = pot2(GG - 30 - sa1);
#pragma unroll 1
                        for (int hf = 0; hf < 4; hf++) {
                            uint32_t d0[8], d1[8];
                            tmem_le8x2(base_h + hf * 8 + t0 * TNv, base_h + hf * 8 + t1 * TNv, d0, d1);
                            const float* tb0 = tb_h + hf * 8;
                            const float* tb1 = tb0 + TNv;
#pragma unroll
                            for (int k = 0; k < 8; k++) {
                                const float f0 = tb0[k], f1 = tb1[k];
                                const uint32_t rap0 = __float_as_uint(fmaf(fmaf(__uint_as_float(d0[k]), fa0, cn0), f0, MAGIA_F));
                                const uint32_t rap1 = __float_as_uint(fmaf(fmaf(__uint_as_float(d1[k]), fa1, cn1), f1, MAGIA_F));
                                const int ex0 = __float2int_rn(((float)((int)d0[k] - DESLOC) * ga0) * f0), ex1 = __float2int_rn(((float)((int)d1[k] - DESLOC) * ga1) * f1);
                                const int dif = (int)((uint32_t)ex0 + MAGIA - rap0) + (int)((uint32_t)ex1 + MAGIA - rap1);
                                // the accumulator is a compile-time register only under full unrolling: select by hf
#pragma unroll
                                for (int g = 0; g < 4; g++) acc[g * 8 + k] += g == hf ? dif : 0;
                            }
                        }
                    }
                    tc_fence_antes();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(bar_tempty + 8 * t0);
                }
                if (!ok) break;
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_bempty + 8 * sl);
                eaw = eaw_prox;
            }
        } else
        for (int c = 0; c < pedacos_por_parte && ok; c++) {
            const int sl = c % NTB;
            if (c + 1 < pedacos_por_parte) eaw_prox = le_exp(c + 1);
            ok = __all_sync(FULL, espera(bar_bfull + 8 * sl, (c / NTB) & 1, aborta, kid, 6));
            if (!ok) break;
            // one tensor-memory stage per K-block of the chunk when both count 4: stage and phase are compile-time per q
            constexpr bool FIXO = NQ == NTM;
#pragma unroll
            for (int q = 0; q < NQ; q++, f++) {
                const int t = FIXO ? q : f % NTM;
                ok = __all_sync(FULL, espera(bar_tfull + 8 * t, (FIXO ? c : f / NTM) & 1, aborta, kid, 4));
                if (!ok) break;
                tc_fence_depois();
                uint32_t d[32];
                tmem_le32(tmem + ((uint32_t)(quarto * 32) << 16) + t * TNv + cg * 32, d);
                tc_fence_antes();
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_tempty + 8 * t);
                const int sa = min(RA - (int)(int8_t)(eaw >> (8 * q)), 40);
                const float fa = pot2(GG - sa), cneg = -MAGIA_F * fa;
                const float4* tb = reinterpret_cast<const float4*>(tabB + (sl * 4 + q) * TNv + cg * 32);
#pragma unroll
                for (int j4 = 0; j4 < 8; j4++) {
                    const float4 fb = tb[j4];
                    const float fbv[4] = {fb.x, fb.y, fb.z, fb.w};
#pragma unroll
                    for (int k = 0; k < 4; k++) {
                        const int j = j4 * 4 + k;
                        const float g = fmaf(__int_as_float((int)(d[j] + MAGIA)), fa, cneg);      // = p * 2^(4 - sa), exact
                        acc[j] += __float2int_rn(g * fbv[k]);
                    }
                }
            }
            if (!ok) break;
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_bempty + 8 * sl);
            eaw = eaw_prox;
        }
        if (PARES) {
            const uint32_t vies = (uint32_t)nfatias * MAGIA;
#pragma unroll
            for (int j = 0; j < 32; j++) acc[j] = (int)((uint32_t)acc[j] - vies);
        }
#pragma unroll
        for (int j = 0; j < 32; j += 4)
            *reinterpret_cast<int4*>(acc_s + lin * PITCHv + cg * 32 + j) = make_int4(acc[j], acc[j + 1], acc[j + 2], acc[j + 3]);
        // the only barrier of the drain warps: reached by every drain thread exactly once, aborted or not
        asm volatile("bar.sync 1, %0;" ::"n"(N_EPI) : "memory");
        epilogo_tile<BLK, MODO, N_EPI, TNv>(acc_s, RAs, RBs, TM, m0, n0, N, S, gridDim.z > 1, blockIdx.z == 0, kid, et, RBf, RBm);
    }
    tc_fence_antes();
    __syncthreads();
    if (wid == 1) {
        tc_fence_depois();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(NTM * TNv) : "memory");
    }
}

}  // namespace tc

// ---------------------------------------------------------------------------------------------- tensor maps (host)
// cuTensorMapEncodeTiled through the runtime's driver entry point (no link against libcuda)
typedef CUresult (*PFN_tmap)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                             const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static PFN_tmap g_tmap = nullptr;
static bool g_tmap_tentou = false;

static PFN_tmap pega_tmap() {
    if (!g_tmap_tentou) {
        g_tmap_tentou = true;
        void* f = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
            g_tmap = (PFN_tmap)f;
    }
    return g_tmap;
}

// 2-D map of an int8 matrix [linhas, K] (K contiguous): box = linhas_caixa rows x 128 bytes, 128-byte swizzle
static bool faz_mapa(CUtensorMap* m, const void* p, int linhas, int K, int linhas_caixa = tc::TM) {
    PFN_tmap f = pega_tmap();
    if (!f) return false;
    cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)linhas};
    cuuint64_t passos[1] = {(cuuint64_t)K};
    cuuint32_t caixa[2] = {(cuuint32_t)tc::KC, (cuuint32_t)linhas_caixa};
    cuuint32_t um[2] = {1, 1};
    return f(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(p), dims, passos, caixa, um, CU_TENSOR_MAP_INTERLEAVE_NONE,
             CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace jt
