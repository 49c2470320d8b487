// CUDA-core block GEMM (dp4a): the path for shapes the tensor-core kernel does not take (rows not a multiple
// of 128) and an independent second implementation of the same arithmetic, selectable with jt_gemm_via(2).
//
// C[M,N] = A[M,K] . B[N,K]^T, operands blocked along K (jatai_cuda/ops.py:95-108): for every K-block the exact
// int8 dot product p is rounded by (RA_i - ea_ib) + (RB_j - eb_jb) after a left shift of GG bits, then added.
// Tile 64 x 128, 256 threads, 4 x 8 outputs per thread, one 32-wide K slice in shared memory per iteration.
#pragma once
#include "gemm_comum.cuh"

namespace jt {

template <int BLK, int MODO>
__global__ void __launch_bounds__(256) k_gemm_simt(const int8_t* __restrict__ A, const int8_t* __restrict__ EA, const int8_t* __restrict__ B,
                                                   const int8_t* __restrict__ EB, const int8_t* __restrict__ RAg, const int8_t* __restrict__ RBg,
                                                   SaidaGemm S, int M, int N, int K, int fatias_por_parte, int kid) {
    constexpr int TM = 64, SUB = BLK / 32;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    uint32_t (*As)[9] = reinterpret_cast<uint32_t (*)[9]>(smem_raw);                          // [TM][9]
    uint32_t (*Bs)[9] = reinterpret_cast<uint32_t (*)[9]>(smem_raw + TM * 9 * 4);              // [TN][9]
    int* RAs = reinterpret_cast<int*>(smem_raw + (TM + TN) * 9 * 4);
    int* RBs = RAs + TM;
    int* acc_s = RBs + TN;                                                                    // [TM][PITCH]
    const int tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;
    const int m0 = blockIdx.y * TM, n0 = blockIdx.x * TN;
    const int nb = K / BLK;
    if (tid < TM) RAs[tid] = RAg ? (int)RAg[m0 + tid] : max_expoentes(EA + (size_t)(m0 + tid) * nb, nb);
    else if (tid < TM + TN) RBs[tid - TM] = RBg ? (int)RBg[n0 + tid - TM] : max_expoentes(EB + (size_t)(n0 + tid - TM) * nb, nb);
    __syncthreads();
    int acc[4][8], p[4][8];
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 8; j++) acc[i][j] = p[i][j] = 0;
    const int f0 = blockIdx.z * fatias_por_parte;            // 32-wide slices [f0, f0 + fatias_por_parte)
    for (int f = f0; f < f0 + fatias_por_parte; f++) {
        __syncthreads();
        if (tid < 128) {
            const int r = tid >> 1, h = tid & 1;
            const uint4 v = *reinterpret_cast<const uint4*>(A + (size_t)(m0 + r) * K + f * 32 + h * 16);
            As[r][h * 4] = v.x; As[r][h * 4 + 1] = v.y; As[r][h * 4 + 2] = v.z; As[r][h * 4 + 3] = v.w;
        }
        {
            const int r = tid >> 1, h = tid & 1;
            const uint4 v = *reinterpret_cast<const uint4*>(B + (size_t)(n0 + r) * K + f * 32 + h * 16);
            Bs[r][h * 4] = v.x; Bs[r][h * 4 + 1] = v.y; Bs[r][h * 4 + 2] = v.z; Bs[r][h * 4 + 3] = v.w;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < 8; kk++) {
            int a4[4], b4[8];
#pragma unroll
            for (int i = 0; i < 4; i++) a4[i] = (int)As[ty * 4 + i][kk];
#pragma unroll
            for (int j = 0; j < 8; j++) b4[j] = (int)Bs[tx * 8 + j][kk];
#pragma unroll
            for (int i = 0; i < 4; i++)
#pragma unroll
                for (int j = 0; j < 8; j++) p[i][j] = __dp4a(a4[i], b4[j], p[i][j]);
        }
        if ((f + 1) % SUB == 0) {                            // a K-block is complete: align, round, add
            const int b = f / SUB;
            int sa[4], sb[8];
#pragma unroll
            for (int i = 0; i < 4; i++) sa[i] = RAs[ty * 4 + i] - (int)EA[(size_t)(m0 + ty * 4 + i) * nb + b];
#pragma unroll
            for (int j = 0; j < 8; j++) sb[j] = RBs[tx * 8 + j] - (int)EB[(size_t)(n0 + tx * 8 + j) * nb + b];
#pragma unroll
            for (int i = 0; i < 4; i++)
#pragma unroll
                for (int j = 0; j < 8; j++) { acc[i][j] += rnd_d(p[i][j] << GG, sa[i] + sb[j]); p[i][j] = 0; }
        }
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < 4; i++) {
        int* d = acc_s + (ty * 4 + i) * PITCH + tx * 8;
        *reinterpret_cast<int4*>(d) = make_int4(acc[i][0], acc[i][1], acc[i][2], acc[i][3]);
        *reinterpret_cast<int4*>(d + 4) = make_int4(acc[i][4], acc[i][5], acc[i][6], acc[i][7]);
    }
    __syncthreads();
    epilogo_tile<BLK, MODO, 256>(acc_s, RAs, RBs, TM, m0, n0, N, S, gridDim.z > 1, blockIdx.z == 0, kid, tid);
}

constexpr int SIMT_SMEM = (64 + TN) * 9 * 4 + (64 + TN) * 4 + 64 * PITCH * 4;

}  // namespace jt
