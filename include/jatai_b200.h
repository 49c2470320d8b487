/* C ABI of libjatai_b200.so: the integer-only (INT8 mantissa + block exponent) training kernels for B200.
 *
 * This is the drop-in boundary.  Every entry point below that cites `jatai_cuda.cu:<line>` has the name,
 * argument order, argument meaning and return convention of the `extern "C"` function at that line of the
 * reference's jatai_cuda/jatai_cuda.cu, which the reference binds with ctypes (jatai_cuda/ops.py:299-324):
 * a launcher written for the reference library works on this one after changing the path it dlopens.
 *
 * Conventions (jatai_cuda.cu:1051-1059, ops.py:313-324):
 *   - pointers are raw device pointers (NULL for an absent tensor); dimensions are C ints; block counts are
 *     long long; the LAST argument of every operation is the launch id `kid`, echoed in the error record;
 *   - the return value is the cudaError_t of the launch as an int: 0 = launched; invalid arguments return
 *     cudaErrorInvalidValue (1) and launch nothing;
 *   - all launches go to the stream given to jt_stream (NULL = legacy default stream); nothing synchronises
 *     except jt_erro_le and jt_sincroniza, so a whole step can be captured in a CUDA graph;
 *   - every input and output is owned by the caller; the only device memory the library allocates is the attention
 *     workspace, one per device: cudaMalloc the first time a size is seen, reused afterwards, replaced by a larger one when
 *     needed (never freed: a recorded CUDA graph may hold the old address; growth inside a stream capture is refused with
 *     cudaErrorStreamCaptureUnsupported, so run one step eagerly before capturing).  Head dimension 64: the split operands
 *     (384 bytes per token and head in the forward, 640 in the backward) and, in the backward, 2*Bt*H*T*T bytes of dS' digits;
 *     other head dimensions: Bt*H*(8+T+T*T) ints (the T*T part only below 1 GiB).  Calls that overlap on the GPU share it;
 *   - host state (stream, block length, paths) is per process; the workspace and kernel attributes are kept per device;
 *   - kernels never trap: a broken invariant is recorded in the device error record and the kernel goes on.
 *
 * Tensor formats (jatai_cuda.cu:3-9):
 *   block tensor: m int8 [R x C] row-major, E int8 [R x C/BLK]; value = m * 2^E; an all-zero block has E = -127;
 *   raw tensor:   acc int32 [R x C], e int16 [R x C] (one exponent per element).
 * BLK is 32 by default (jt_blk); 128 is the reference's format.
 */
#ifndef JATAI_B200_H
#define JATAI_B200_H

#ifdef __cplusplus
extern "C" {
#endif

/* ---- device error record and control --------------------------------------------------------------- */
/* out[0..5] = n events, code, kid, flat index into the output, value, extra.  Returns n, or -cudaError.
 * Synchronises.  Codes 1..6 as in the reference (jatai_cuda.cu:22), 7 = a bounded in-kernel wait expired.
 * jatai_cuda.cu:1062 */
int jt_erro_le(long long* out);
int jt_erro_limpa(void);                                   /* jatai_cuda.cu:1069 */
int jt_sincroniza(void);                                   /* jatai_cuda.cu:1073 */
void jt_stream(void* cuda_stream);                         /* jatai_cuda.cu:1088 */
void jt_gemm_split(int alvo_ctas);                         /* jatai_cuda.cu:1089: split-K target (CTAs) of raw GEMMs */
void jt_gemm_bm(int bm);                                   /* jatai_cuda.cu:1090: accepted, ignored (tile height is fixed) */
void jt_atencao_linhas(int n);                             /* jatai_cuda.cu:1091: accepted, ignored */
int jt_res_estocastico(int ligado);                        /* jatai_cuda.cu:1087: only 0 is supported (bit parity) */
/* No counterpart in the reference (its kernels never wait on one another).  Every wait of the tensor-core kernels on an
 * mbarrier is bounded; jt_espera_limite sets the bound in SM clock cycles (<= 0: the default, about 2 s).  jt_teste_espera
 * runs the bounded wait on its own - one warp, a barrier that nothing completes, no copy or MMA in flight - so that the
 * give-up path can be exercised with a short limit: *saiu (a device int) becomes 2 and the error record holds code 7,
 * place 99; the context stays usable. */
int jt_espera_limite(long long ciclos);
/* No counterpart in the reference.  1: the kernels of the training step are launched as programmatic dependent launches -
 * each may be scheduled while its predecessor in the stream drains and waits (griddepcontrol.wait) before its first access
 * to global memory; 0 (default): plain stream order.  Same results either way. */
int jt_pdl(int ligado);
int jt_teste_espera(int* saiu, int kid);
/* Test switch, no counterpart in the reference: 1 = the tensor-core GEMM issues no operand load; its first in-kernel wait
 * then runs out after the limit in force with no copy or MMA in flight, every warp leaves through the abort path, the
 * launch returns with code 7 recorded (outputs undefined).  0 = normal. */
int jt_gemm_sem_cargas(int ligado);

/* ---- GEMM: C[M,N] = A[M,K] . B[N,K]^T, operands blocked along K ---------------------------------- */
/* modo 0 block output (Cm, CE) | 1 raw output (C32, Ce) | 2 block + residual add of X | 3 block h and
 * Om2/OE2 = relu2(h) | 4 relu2_back(A.B^T, X).  M multiple of 64, N of 128, K of BLK.
 * jatai_cuda.cu:1093 */
int jt_gemm_f(const void* A, const void* EA, const void* B, const void* EB, void* Cm, void* CE, void* C32, void* Ce,
              const void* Xm, const void* XE, void* Om2, void* OE2, int M, int N, int K, int modo, int kid);
/* jatai_cuda.cu:1124 */
int jt_gemm(const void* A, const void* EA, const void* B, const void* EB, void* Cm, void* CE, void* C32, void* Ce,
            int M, int N, int K, int modo, int kid);

/* ---- block operations ---------------------------------------------------------------------------- */
int jt_quant(const void* acc, const void* e, void* m, void* E, long long nblocos, int kid);                     /* jatai_cuda.cu:1128 */
int jt_soma(const void* xm, const void* xE, const void* ym, const void* yE, void* zm, void* zE,
            long long nblocos, int kid);                                                                        /* jatai_cuda.cu:1132 */
int jt_relu2(const void* hm, const void* hE, void* am, void* aE, long long nblocos, int kid);                   /* jatai_cuda.cu:1137 */
int jt_relu2_back(const void* gm, const void* gE, const void* hm, const void* hE, void* om, void* oE,
                  long long nblocos, int kid);                                                                  /* jatai_cuda.cu:1141 */
int jt_momento(const void* gacc, const void* ge, void* Mm, void* ME, long long nblocos, int kid);               /* jatai_cuda.cu:1146 */
int jt_peso(void* Wm, void* WE, const void* Mm, const void* ME, void* Rm, void* RE, int k_lr, int ef,
            long long nblocos, int kid);                                                                        /* jatai_cuda.cu:1150 */
int jt_transpoe(const void* X, const void* EX, void* Y, void* EY, int R, int C, int kid);                       /* jatai_cuda.cu:1155 */
int jt_embed(const void* Wm, const void* WE, const void* tok, void* Xm, void* XE, int M, int D, int V, int kid); /* jatai_cuda.cu:1159 */
int jt_um_quente(const void* tok, void* U, void* UE, int M, int V, int kid);                                    /* jatai_cuda.cu:1163 */
int jt_rms(const void* Xm, const void* XE, void* Ym, void* YE, void* cr, void* cemax, int M, int D, int log2D,
           int G, int kid);                                                                                     /* jatai_cuda.cu:1167 */
int jt_rms_back(const void* gm, const void* gE, const void* ym, const void* yE, const void* cr, const void* cemax,
                void* om, void* oE, int M, int D, int log2D, int G, int GB, int kid);                           /* jatai_cuda.cu:1171 */
/* QKV is one block tensor [Bt*T, 3D] (q | k | v); Oacc/Oe raw [Bt*T, D]; P uint8 [Bt*H][T][T] stored key-major.
 * Head dimension D/H in {4, 16, 64}; T a multiple of 32, at most 1024.  jatai_cuda.cu:1177 */
int jt_atencao(const void* qm, const void* qE, void* Oacc, void* Oe, void* P, int Bt, int T, int H, int D, int GA, int kid);
/* Gacc/Ge raw [Bt*T, 3D] (gq | gk | gv).  jatai_cuda.cu:1182 */
int jt_atencao_back(const void* gom, const void* goE, const void* qm, const void* qE, const void* P, void* Gacc, void* Ge,
                    int Bt, int T, int H, int D, int GA, int limite, int kid);
int jt_softmax_ce(const void* acc, const void* e, const void* alvo, void* gm, void* gE, void* d_alvo, void* soma,
                  int M, int V, int log2M, int kid);                                                            /* jatai_cuda.cu:1195 */

/* The reference's 16-bit residual stream (opt-in ablation, no int64 specification).  Exported so that a launcher
 * that looks the symbols up keeps working; each returns cudaErrorNotSupported.  jatai_cuda.cu:1074-1086 */
int jt_para16(const void* xm, const void* xE, void* zm, void* zE, long long nblocos, int kid);
int jt_para8(const void* xm, const void* xE, void* ym, void* yE, long long nblocos, int kid);
int jt_soma16(const void* xm, const void* xE, const void* ym, const void* yE, void* zm, void* zE, long long nblocos, int kid);

/* ---- additions of this library (no counterpart in the reference) --------------------------------- */
/* Exponent block length used by every later call: 32 (default) or 128 (the reference's compile-time BLK,
 * jatai_cuda.cu:16).  Host state, like jt_stream. */
int jt_blk(int blk);
int jt_blk_atual(void);
/* GEMM path: 0 automatic | 1 tensor cores, refused (cudaErrorInvalidValue) on a shape they do not take | 2 CUDA cores (dp4a) |
 * 3 tensor cores with every K-block rounded by a float-to-int conversion (block 32's default rounds with an FMA against
 * 1.5*2^23 after a range check, and converts only the columns that fail it; both are exact for every input). */
int jt_gemm_via(int via);
/* jt_quant(jt_atencao(...)) / jt_quant(jt_atencao_back(...)) with the quantisation done in the attention kernels' output stage:
 * Om, OE = block tensor [Bt*T, D]; Gm, GE = block tensor [Bt*T, 3D] (gq | gk | gv); other arguments as in jt_atencao /
 * jt_atencao_back.  Same results as the two calls.  Served at block length 32, head dimension 64, T >= 128 (the tensor-core
 * path); cudaErrorNotSupported (801) elsewhere - compose the two calls then. */
int jt_atencao_quant(const void* qm, const void* qE, void* Om, void* OE, void* P, int Bt, int T, int H, int D, int GA, int kid);
int jt_atencao_back_quant(const void* gom, const void* goE, const void* qm, const void* qE, const void* P, void* Gm, void* GE,
                          int Bt, int T, int H, int D, int GA, int limite, int kid);
/* Attention path: 0 automatic (tensor cores when the head dimension is 64 and T >= 128; one CTA per head when T <= 128 and the
 * head dimension is 4 or 16) | 1 the tiled CUDA-core kernels.  Same bits either way. */
int jt_atencao_via(int via);
/* Tile width of the tensor-core GEMM: 0 automatic (64 columns when 128-column tiles would leave most SMs idle, block
 * 32 only) | 64 | 128. */
int jt_gemm_tn(int tn);
/* jt_gemm_f with optional externally supplied row-maximum exponents RA[M], RB[N] (int8).  A data-parallel rank
 * passes the maxima over all ranks, so that the int32 partial sums of all ranks share one exponent and their
 * integer sum equals the single-GPU result (the reference's split-K argument, jatai_cuda.cu:214-216). */
int jt_gemm_ext(const void* A, const void* EA, const void* B, const void* EB, void* Cm, void* CE, void* C32, void* Ce,
                const void* Xm, const void* XE, void* Om2, void* OE2, const void* RA, const void* RB,
                int M, int N, int K, int modo, int kid);
/* R8[i] = max over the nb block exponents of row i of E (int8 [linhas, nb]): the RA / RB above. */
int jt_max_linha(const void* E, void* R8, int linhas, int nb, int kid);

/* jt_momento followed by jt_peso on the same tensors in one launch (the optimiser step of a weight is always this pair):
 * same results as the two calls, one pass over the momentum.  Arguments as in jt_momento and jt_peso. */
int jt_momento_peso(const void* gacc, const void* ge, void* Mm, void* ME, void* Wm, void* WE, void* Rm, void* RE, int k_lr, int ef,
                    long long nblocos, int kid);

/* jt_soma(x, jt_rms_back(g, y, cache)) in one launch: the residual add that always follows the RMSNorm backward.  x is a
 * block tensor [M, D]; the other arguments as in jt_rms_back.  Same results as the two calls. */
int jt_rms_back_soma(const void* gm, const void* gE, const void* ym, const void* yE, const void* cr, const void* cemax, const void* xm,
                     const void* xE, void* om, void* oE, int M, int D, int log2D, int G, int GB, int kid);

/* Two jt_transpoe calls on matrices with the same row count R ([R, C1] and [R, C2]) in one launch: the two operands of
 * a weight-gradient GEMM.  Same results as the two calls. */
int jt_transpoe2(const void* X1, const void* EX1, void* Y1, void* EY1, const void* X2, const void* EX2, void* Y2, void* EY2, int C1, int C2,
                 int R, int kid);
/* The same, and jt_max_linha of both results: RM1 [C1] and RM2 [C2] (int8, 4-byte aligned, PRE-SET TO -128 BY THE CALLER)
 * receive the largest block exponent of every row of Y1 / Y2 (maximum into what is there).  Data parallel uses it to have
 * the row maxima of its weight-gradient operands written straight into the buffer of the MAX collective.  Block 32 and
 * C1, C2 multiples of 256 only (cudaErrorNotSupported otherwise: call jt_transpoe2 and jt_max_linha).  No counterpart in
 * the reference. */
int jt_transpoe2_max(const void* X1, const void* EX1, void* Y1, void* EY1, const void* X2, const void* EX2, void* Y2, void* EY2, void* RM1,
                     void* RM2, int C1, int C2, int R, int kid);

/* jt_atencao_back for callers that may not allocate device memory (fixed memory budgets, code running where
 * cudaMalloc is forbidden): same arguments and results, but the workspace lives in a fixed 4 MiB device array
 * inside the library instead of a cudaMalloc'd buffer, and no allocating routine is called.  Refuses
 * Bt*H*(8+T) > 2^20 with cudaErrorInvalidValue; when Bt*H*(8+T+T*T) does not fit either, its kernels recompute the
 * intermediate matrices instead of handing them on (same bits, slower).  The first call on a device resolves the array's address: make it
 * outside stream capture.  All calls share the array; calls that overlap on the GPU race.
 * It has no counterpart in the reference. */
int jt_atencao_back_fixo(const void* gom, const void* goE, const void* qm, const void* qE, const void* P, void* Gacc, void* Ge,
                         int Bt, int T, int H, int D, int GA, int limite, int kid);

#ifdef __cplusplus
}
#endif
#endif
