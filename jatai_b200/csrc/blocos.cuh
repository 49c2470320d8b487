// Bandwidth-bound block kernels: quant, soma, relu2(+back), momento, peso, embed, um_quente, transpoe,
// rms(+back), softmax_ce.  One pass over HBM each, 128-bit accesses.
//
// Work decomposition (all kernels): one thread owns 16 consecutive elements of a row = one 128-bit load of
// int8 mantissas; GL = BLK/16 neighbouring lanes own one exponent block and reduce with xor-shuffles.
// Arithmetic: the int64 specification of the reference (jatai_cuda/ops.py, cited per kernel) in int32.
#pragma once
#include "comum.cuh"

namespace jt {

#define JT_FIO16                                                                         \
    const long long t_ = (long long)blockIdx.x * blockDim.x + threadIdx.x;               \
    const bool ativo = t_ < n16;                                                         \
    const long long t16 = ativo ? t_ : 0;   /* idle lanes recompute thread 0, store nothing */ \
    const long long o = t16 * 16;                                                        \
    const long long w = o / BLK;                                                         \
    const bool lider = ativo && (t16 % (BLK / 16) == 0);

// raw (acc int32, e int16 per element) -> block.  ops.py:125-126
template <int BLK>
__global__ void __launch_bounds__(256) k_quant(const int* __restrict__ acc, const int16_t* __restrict__ e, int8_t* __restrict__ m,
                                               int8_t* __restrict__ E, long long n16, int kid) {
    JT_FIO16
    int v[16], ee[16], q[16];
    le16_i32(acc + o, v);
    le16_i16(e + o, ee);
    {
        // fp32 path (a whole warp or none): every |v| <= 2^24 is exact in fp32, v * 2^(e - largest exponent of a non-zero value
        // of the block) is an exact scaling while the exponents are at most 100 apart, and the fp32 quantiser then gives the
        // bits of the integer one (the block's top bit and the one-more-bit retry depend on the largest scaled magnitude alone)
        int eref = -32768, big = 0;
#pragma unroll
        for (int i = 0; i < 16; i++) {
            big |= (v[i] > (1 << 24)) | (v[i] < -(1 << 24));
            if (v[i] != 0) eref = max(eref, ee[i]);
        }
        eref = grupo_max<BLK / 16>(eref);
#pragma unroll
        for (int i = 0; i < 16; i++) big |= (v[i] != 0) & (eref - ee[i] > 100);
        if (__all_sync(FULL, big == 0)) {
            float f[16];
#pragma unroll
            for (int i = 0; i < 16; i++) f[i] = (float)v[i] * __int_as_float((127 + max(min(ee[i] - eref, 0), -100)) << 23);
            uint4 pac;
            const int Eo = quant_f32<BLK / 16>(f, eref, pac, kid, o);
            if (ativo) *reinterpret_cast<uint4*>(m + o) = pac;
            if (lider) E[w] = (int8_t)Eo;
            return;
        }
    }
    // blocks whose elements all carry one exponent (attention outputs: one exponent per head) take the cheaper
    // uniform quantiser; the choice is made per block, the lanes of a block always agree
    int dif = 0;
#pragma unroll
    for (int i = 1; i < 16; i++) dif |= ee[i] ^ ee[0];
    dif |= ee[0] ^ __shfl_sync(FULL, ee[0], (threadIdx.x & 31) & ~(BLK / 16 - 1));
    dif = grupo_or<BLK / 16>(dif);
    const unsigned m_uni = __ballot_sync(FULL, dif == 0);
    int Eo;
    if (dif == 0) Eo = quant_uniforme<16, BLK / 16>(v, ee[0], q, kid, o, m_uni);
    else Eo = quant_geral<16, BLK / 16>(v, ee, q, kid, o, ~m_uni);
    if (ativo) grava16(m + o, q);
    if (lider) E[w] = (int8_t)Eo;
}

// ---- several 16-element chunks per thread --------------------------------------------------------------
// A thread issues the 128-bit loads of U chunks (one every gridDim*blockDim chunks, so lane groups stay aligned)
// before it touches any of them: with one chunk per thread the ~1300 resident threads of an SM keep only ~20 KB in
// flight, far less than the ~45 KB that HBM latency x bandwidth asks for.
#define JT_PEDACO(k)                                                                      \
    const long long tk_ = t0_ + (long long)(k) * nth_;                                    \
    const bool ativo = tk_ < n16;                                                         \
    const long long t16 = ativo ? tk_ : 0;                                                \
    const long long o = t16 * 16;                                                         \
    const long long w = o / BLK;                                                          \
    const bool lider = ativo && (t16 % (BLK / 16) == 0);
#define JT_MULTI                                                                          \
    const long long nth_ = (long long)gridDim.x * blockDim.x;                             \
    const long long t0_ = (long long)blockIdx.x * blockDim.x + threadIdx.x;

// One 16-element chunk of z = x + y (see k_soma below for the arithmetic); the GL lanes of a block call together.
// Returns the block exponent, `pac` receives the 16 mantissas.
template <int GL>
__device__ __forceinline__ int soma16(const int (&xv)[16], int ex, const int (&yv)[16], int ey, uint4& pac, int kid, long long o) {
    const bool x_maior = ex >= ey;
    const int eH = x_maior ? ex : ey, d = x_maior ? ex - ey : ey - ex;
    const int dl = min(d, 21), s2 = d - dl;                         // s2 > 0: the far operand is rounded first
    int hi[16], lo[16], wv[16];
#pragma unroll
    for (int i = 0; i < 16; i++) { hi[i] = x_maior ? xv[i] : yv[i]; lo[i] = x_maior ? yv[i] : xv[i]; }
    int mx = 0;
#pragma unroll
    for (int i = 0; i < 16; i++) {
        wv[i] = (hi[i] << dl) + rnd_d(lo[i], s2);
        mx = max(mx, wv[i] < 0 ? -wv[i] : wv[i]);
    }
    mx = grupo_max<GL>(mx);
    int s = bitlen(mx) - 7;
    if (desloca(mx, s) > 127) s += 1;
    const int E = eH - dl + s;
    pac = make_uint4(0, 0, 0, 0);
    int Eo = E_ZERO;
    if (mx != 0 && E >= -126) {
        if (E > 126) reporta(E_EXP, kid, o, E, eH);
        Eo = E;
        int q[16];
        if (s > 0) {
            const int c = (1 << (s - 1)) - 1;
#pragma unroll
            for (int i = 0; i < 16; i++) q[i] = (wv[i] + c + ((wv[i] >> s) & 1)) >> s;
        } else {
#pragma unroll
            for (int i = 0; i < 16; i++) q[i] = wv[i] << (-s);
        }
        pac.x = junta4(q[0], q[1], q[2], q[3]);
        pac.y = junta4(q[4], q[5], q[6], q[7]);
        pac.z = junta4(q[8], q[9], q[10], q[11]);
        pac.w = junta4(q[12], q[13], q[14], q[15]);
    }
    return Eo;
}

// z = x + y.  ops.py:128-132: ec = max(xE, yE) - 21; v = rnd(x, ec - xE) + rnd(y, ec - yE); quant(v, ec).
// With hi / lo = the operand of larger / smaller exponent and d their distance, v = 2^(21-dl) * w where dl = min(d, 21),
// w = hi * 2^dl + lo' and lo' = lo (d <= 21) or rnd(lo, d - 21) (the specification rounds the far operand first).
// The quantiser is invariant under the common power of two, so the block is quant(w, e_hi - dl): the same bits with
// 28-bit instead of 30-bit intermediates, one code path for every d, and rounding shifts shared by the block.
template <int BLK, int U = 4>
__global__ void __launch_bounds__(256) k_soma(const int8_t* __restrict__ xm, const int8_t* __restrict__ xE, const int8_t* __restrict__ ym,
                                              const int8_t* __restrict__ yE, int8_t* __restrict__ zm, int8_t* __restrict__ zE,
                                              long long n16, int kid) {
    constexpr int GL = BLK / 16;
    JT_MULTI
    uint4 rx[U], ry[U];
    int ex[U], ey[U];
#pragma unroll
    for (int k = 0; k < U; k++) {
        JT_PEDACO(k)
        rx[k] = *reinterpret_cast<const uint4*>(xm + o);
        ry[k] = *reinterpret_cast<const uint4*>(ym + o);
        ex[k] = xE[w];
        ey[k] = yE[w];
        (void)lider;
    }
#pragma unroll
    for (int k = 0; k < U; k++) {
        JT_PEDACO(k)
        uint4 pac;
        int Eo;
        // fp32 path: with the exponents at most 16 apart w = hi * 2^d + lo is below 2^24, exact in fp32, and the fp32 quantiser
        // gives the bits of the integer one; an all-zero block on either side leaves the other operand alone.  Taken by a
        // whole warp or not at all (the quantisers shuffle inside the lane groups of a block).
        const bool x_maior = ex[k] >= ey[k];
        const int eH = x_maior ? ex[k] : ey[k], eL = x_maior ? ey[k] : ex[k];
        const uint4 rl = x_maior ? ry[k] : rx[k];
        const int d = (eL == E_ZERO && (rl.x | rl.y | rl.z | rl.w) == 0) ? 0 : eH - eL;
        if (__all_sync(FULL, d <= 16)) {
            float fx[16], fy[16];
            bytes_para_float(rx[k], fx);
            bytes_para_float(ry[k], fy);
            const float a = x_maior ? __int_as_float((127 + d) << 23) : 1.f, b = x_maior ? 1.f : __int_as_float((127 + d) << 23);
#pragma unroll
            for (int i = 0; i < 16; i++) fx[i] = fmaf(fx[i], a, fy[i] * b);
            Eo = quant_f32<GL>(fx, eH - d, pac, kid, o);
        } else {
            int xv[16], yv[16];
            desempacota16(rx[k], xv);
            desempacota16(ry[k], yv);
            Eo = soma16<GL>(xv, ex[k], yv, ey[k], pac, kid, o);
        }
        if (ativo) *reinterpret_cast<uint4*>(zm + o) = pac;
        if (lider) zE[w] = (int8_t)Eo;
    }
}

// a = max(h, 0)^2.  ops.py:134-137.  fp32 path: h^2 <= 16129 is exact
template <int BLK, int U = 4>
__global__ void __launch_bounds__(256) k_relu2(const int8_t* __restrict__ hm, const int8_t* __restrict__ hE, int8_t* __restrict__ am,
                                               int8_t* __restrict__ aE, long long n16, int kid) {
    JT_MULTI
    uint4 rh[U];
    int eh[U];
#pragma unroll
    for (int k = 0; k < U; k++) {
        JT_PEDACO(k)
        rh[k] = *reinterpret_cast<const uint4*>(hm + o);
        eh[k] = hE[w];
        (void)lider;
    }
#pragma unroll
    for (int k = 0; k < U; k++) {
        JT_PEDACO(k)
        float f[16];
        bytes_para_float(rh[k], f);
#pragma unroll
        for (int i = 0; i < 16; i++) { const float r = fmaxf(f[i], 0.f); f[i] = r * r; }
        uint4 pac;
        const int Eo = quant_f32<BLK / 16>(f, 2 * eh[k], pac, kid, o);
        if (ativo) *reinterpret_cast<uint4*>(am + o) = pac;
        if (lider) aE[w] = (int8_t)Eo;
    }
}

// gh = g * 2 * max(h, 0).  ops.py:139-141.  fp32 path: |g h 2| <= 32258 is exact
template <int BLK, int U = 4>
__global__ void __launch_bounds__(256) k_relu2_back(const int8_t* __restrict__ gm, const int8_t* __restrict__ gE, const int8_t* __restrict__ hm,
                                                    const int8_t* __restrict__ hE, int8_t* __restrict__ om, int8_t* __restrict__ oE,
                                                    long long n16, int kid) {
    JT_MULTI
    uint4 rg[U], rh[U];
    int ee[U];
#pragma unroll
    for (int k = 0; k < U; k++) {
        JT_PEDACO(k)
        rg[k] = *reinterpret_cast<const uint4*>(gm + o);
        rh[k] = *reinterpret_cast<const uint4*>(hm + o);
        ee[k] = (int)gE[w] + (int)hE[w];
        (void)lider;
    }
#pragma unroll
    for (int k = 0; k < U; k++) {
        JT_PEDACO(k)
        float g[16], h[16];
        bytes_para_float(rg[k], g);
        bytes_para_float(rh[k], h);
#pragma unroll
        for (int i = 0; i < 16; i++) g[i] = g[i] * fmaxf(h[i], 0.f) * 2.f;
        uint4 pac;
        const int Eo = quant_f32<BLK / 16>(g, ee[k], pac, kid, o);
        if (ativo) *reinterpret_cast<uint4*>(om + o) = pac;
        if (lider) oE[w] = (int8_t)Eo;
    }
}

// momentum, in place: m <- quant(rnd(7 m, ec - em) + rnd(g, ec - eg), ec), em = ME - 3,
// per element ec = max(em + 10, eg + bitlen(g)) - 28.  ops.py:273-278
template <int BLK>
__global__ void __launch_bounds__(256) k_momento(const int* __restrict__ gacc, const int16_t* __restrict__ ge, int8_t* __restrict__ Mm,
                                                 int8_t* __restrict__ ME, long long n16, int kid) {
    JT_FIO16
    int mm[16], g[16], eg[16], v[16], ee[16], q[16];
    le16(Mm + o, mm);
    le16_i32(gacc + o, g);
    le16_i16(ge + o, eg);
    const int em = (int)ME[w] - 3;
#pragma unroll
    for (int i = 0; i < 16; i++) {
        if (g[i] >= LIM || g[i] <= -LIM) reporta(E_ACUM, kid, o + i, g[i], eg[i]);
        const int ec = max(em + 10, eg[i] + bitlen(g[i])) - 28;
        // left shifts cannot lose bits here: |7 m| < 2^10 moves up by at most 18, g by at most 28 - bitlen(g)
        v[i] = desloca(mm[i] * 7, ec - em) + desloca(g[i], ec - eg[i]);
        ee[i] = ec;
    }
    const int Eo = quant_geral<16, BLK / 16>(v, ee, q, kid, o);
    if (ativo) grava16(Mm + o, q);
    if (lider) ME[w] = (int8_t)Eo;
}

// weight step with error feedback, in place on W and R.  ops.py:280-290
template <int BLK>
__global__ void __launch_bounds__(256) k_peso(int8_t* __restrict__ Wm, int8_t* __restrict__ WE, const int8_t* __restrict__ Mm,
                                              const int8_t* __restrict__ ME, int8_t* __restrict__ Rm, int8_t* __restrict__ RE, int k_lr, int ef,
                                              long long n16, int kid) {
    JT_FIO16
    int wv[16], mv[16], rv[16], alvo[16], q[16];
    le16(Wm + o, wv);
    le16(Mm + o, mv);
    if (ef) le16(Rm + o, rv);
    else {
#pragma unroll
        for (int i = 0; i < 16; i++) rv[i] = 0;
    }
    const int ew = WE[w], em = (int)ME[w] - k_lr, er = ef ? (int)RE[w] : E_ZERO;
    const int ec = max(max(ew + 7, em + 7), er + 7) - 27;
    // every operand is a mantissa (7 bits) moved up by at most 20: the left shifts cannot lose bits
#pragma unroll
    for (int i = 0; i < 16; i++)
        alvo[i] = desloca(wv[i], ec - ew) - desloca(mv[i], ec - em) + (ef ? desloca(rv[i], ec - er) : 0);
    const int Ew = quant_uniforme<16, BLK / 16>(alvo, ec, q, kid, o);
    if (ativo) grava16(Wm + o, q);
    if (lider) WE[w] = (int8_t)Ew;
    if (!ef) return;
    int dif[16], r[16];
#pragma unroll
    for (int i = 0; i < 16; i++) dif[i] = alvo[i] - desloca(q[i], ec - Ew);          // q 2^(Ew - ec) stays below the 2^30 of alvo's range
    const int Er = quant_uniforme<16, BLK / 16>(dif, ec, r, kid, o);
    if (ativo) grava16(Rm + o, r);
    if (lider) RE[w] = (int8_t)Er;
}

// momentum and weight step of the same 16 elements in one launch (the optimiser of a weight is always this pair):
// k_momento followed by k_peso on the momentum just written, which stays in registers.
template <int BLK>
__global__ void __launch_bounds__(256) k_momento_peso(const int* __restrict__ gacc, const int16_t* __restrict__ ge, int8_t* __restrict__ Mm,
                                                      int8_t* __restrict__ ME, int8_t* __restrict__ Wm, int8_t* __restrict__ WE,
                                                      int8_t* __restrict__ Rm, int8_t* __restrict__ RE, int k_lr, int ef, long long n16, int kid) {
    pdl_espera();
    pdl_solta();
    JT_FIO16
    int mv[16], Em;
    {
        int mm[16], g[16], eg[16], v[16], ee[16];
        le16(Mm + o, mm);
        le16_i32(gacc + o, g);
        le16_i16(ge + o, eg);
        const int em = (int)ME[w] - 3;
#pragma unroll
        for (int i = 0; i < 16; i++) {
            if (g[i] >= LIM || g[i] <= -LIM) reporta(E_ACUM, kid, o + i, g[i], eg[i]);
            const int ec = max(em + 10, eg[i] + bitlen(g[i])) - 28;
            v[i] = desloca(mm[i] * 7, ec - em) + desloca(g[i], ec - eg[i]);
            ee[i] = ec;
        }
        Em = (int)(int8_t)quant_geral<16, BLK / 16>(v, ee, mv, kid, o);
        if (ativo) grava16(Mm + o, mv);
        if (lider) ME[w] = (int8_t)Em;
    }
    int wv[16], rv[16], alvo[16], q[16];
    le16(Wm + o, wv);
    if (ef) le16(Rm + o, rv);
    else {
#pragma unroll
        for (int i = 0; i < 16; i++) rv[i] = 0;
    }
    const int ew = WE[w], em = Em - k_lr, er = ef ? (int)RE[w] : E_ZERO;
    const int ec = max(max(ew + 7, em + 7), er + 7) - 27;
#pragma unroll
    for (int i = 0; i < 16; i++)
        alvo[i] = desloca(wv[i], ec - ew) - desloca(mv[i], ec - em) + (ef ? desloca(rv[i], ec - er) : 0);
    const int Ew = quant_uniforme<16, BLK / 16>(alvo, ec, q, kid, o);
    if (ativo) grava16(Wm + o, q);
    if (lider) WE[w] = (int8_t)Ew;
    if (!ef) return;
    int dif[16], r[16];
#pragma unroll
    for (int i = 0; i < 16; i++) dif[i] = alvo[i] - desloca(q[i], ec - Ew);
    const int Er = quant_uniforme<16, BLK / 16>(dif, ec, r, kid, o);
    if (ativo) grava16(Rm + o, r);
    if (lider) RE[w] = (int8_t)Er;
}

// row gather of the embedding table; an out-of-range token zeroes the row and records E_ARG.  ops.py:143-145
template <int BLK>
__global__ void __launch_bounds__(256) k_embed(const int8_t* __restrict__ Wm, const int8_t* __restrict__ WE, const int* __restrict__ tok,
                                               int8_t* __restrict__ Xm, int8_t* __restrict__ XE, int M, int D, int V, int kid) {
    pdl_espera();
    pdl_solta();
    const int por_linha = D / 16;
    const long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= (long long)M * por_linha) return;
    const int lin = (int)(t / por_linha), c = (int)(t % por_linha) * 16;
    const int tk = tok[lin];
    const bool ok = tk >= 0 && tk < V;
    if (!ok && c == 0) reporta(E_ARG, kid, (long long)lin * D, tk, V);
    uint4 v = make_uint4(0, 0, 0, 0);
    if (ok) v = *reinterpret_cast<const uint4*>(Wm + (size_t)tk * D + c);
    *reinterpret_cast<uint4*>(Xm + (size_t)lin * D + c) = v;
    if (c % BLK == 0) XE[(size_t)lin * (D / BLK) + c / BLK] = ok ? WE[(size_t)tk * (D / BLK) + c / BLK] : (int8_t)E_ZERO;
}

// one-hot rows with exponent 0 (the embedding gradient is a GEMM on them).  ops.py:147-151
template <int BLK>
__global__ void __launch_bounds__(256) k_um_quente(const int* __restrict__ tok, int8_t* __restrict__ U, int8_t* __restrict__ UE, int M, int V,
                                                   int kid) {
    pdl_espera();
    pdl_solta();
    const int por_linha = V / 16;
    const long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= (long long)M * por_linha) return;
    const int lin = (int)(t / por_linha), c = (int)(t % por_linha) * 16;
    const int tk = tok[lin];
    if ((tk < 0 || tk >= V) && c == 0) reporta(E_ARG, kid, (long long)lin * V, tk, V);
    uint32_t u[4] = {0, 0, 0, 0};
    if (tk >= c && tk < c + 16) u[(tk - c) >> 2] = 1u << (8 * ((tk - c) & 3));
    *reinterpret_cast<uint4*>(U + (size_t)lin * V + c) = make_uint4(u[0], u[1], u[2], u[3]);
    if (c % BLK == 0) UE[(size_t)lin * (V / BLK) + c / BLK] = 0;
}

// [R,C] blocked along C -> [C,R] blocked along R; the new blocks span BLK rows of one column, so every
// element brings its own exponent and the block is quantised again.  ops.py:121-123
// Tile: 128 rows x 64 columns through shared memory; a thread then owns 16 consecutive rows of one column.
template <int BLK>
__global__ void __launch_bounds__(256) k_transpoe(const int8_t* __restrict__ X, const int8_t* __restrict__ EX, int8_t* __restrict__ Y,
                                                  int8_t* __restrict__ EY, int R, int C, int kid) {
    constexpr int TR = 128, TC = 64, NE = (TC + BLK - 1) / BLK;     // exponent columns a tile touches
    __shared__ int8_t tile[TC][TR + 16];                            // stored transposed: [column][row]
    __shared__ int8_t et[TR][NE];
    const int r0 = blockIdx.y * TR, c0 = blockIdx.x * TC;
    const int tid = threadIdx.x;
    // load: 128 rows x 64 B = 512 x 16 B, two per thread, scattered transposed into shared memory
#pragma unroll
    for (int it = 0; it < 2; it++) {
        const int idx = tid + it * 256, lr = idx / 4, lc = (idx % 4) * 16;
        const uint4 v = *reinterpret_cast<const uint4*>(X + (size_t)(r0 + lr) * C + c0 + lc);
        const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int k = 0; k < 16; k++) tile[lc + k][lr] = (int8_t)(u[k >> 2] >> (8 * (k & 3)));
    }
    for (int i = tid; i < TR * NE; i += 256) et[i / NE][i % NE] = EX[(size_t)(r0 + i / NE) * (C / BLK) + c0 / BLK + i % NE];
    __syncthreads();
    // 64 columns x 8 row-groups of 16 = 512 tasks; consecutive lanes take consecutive row-groups of a column
#pragma unroll
    for (int it = 0; it < 2; it++) {
        const int idx = tid + it * 256, col = idx / 8, rg = idx % 8;
        int v[16], e[16], q[16];
        const uint4 w4 = *reinterpret_cast<const uint4*>(&tile[col][rg * 16]);
        const uint32_t u[4] = {w4.x, w4.y, w4.z, w4.w};
#pragma unroll
        for (int k = 0; k < 16; k++) {
            v[k] = (int)(int8_t)(u[k >> 2] >> (8 * (k & 3)));
            e[k] = et[rg * 16 + k][(c0 % BLK + col) / BLK];
        }
        const long long o = (long long)(c0 + col) * R + r0 + rg * 16;
        const int Eo = quant_geral<16, BLK / 16>(v, e, q, kid, o);
        grava16(Y + o, q);
        if (rg % (BLK / 16) == 0) EY[(size_t)(c0 + col) * (R / BLK) + (r0 + rg * 16) / BLK] = (int8_t)Eo;
    }
}

// Transposition for block 32, wide tiles: TR (32, 64 or 128) rows x 256 columns per CTA of 2 TR threads; the launcher
// takes the tallest tile that still gives every SM a CTA (and, for the smallest matrices, a thread per column instead
// of per word: CPT = 1).  A thread owns a 32-row block of 4
// adjacent columns (one 32-bit word per row) and quantises the 4 new blocks without leaving its registers.
// The quantiser runs in fp32, exactly: a mantissa times 2^(e - eref) is exact in fp32, the largest magnitude gives
// top = max(e + bitlen(v)) through its exponent field, and one FFMA against 1.5*2^23 rounds v * 2^(e - E) half to
// even (|result| <= 127, inside the window).  A transposed block can never need the "one more bit" retry
// (|m| <= 127 going in).  Blocks whose exponents are more than 100 apart take an integer path.
constexpr int T32_PW = 256 / 4 + 1;
// integer path of k_transpoe32 for one column of a block whose exponents are too far apart for fp32 (cold)
__device__ __noinline__ int transpoe32_lento(const uint32_t (*tile)[T32_PW], const int8_t (*et)[8], int rb, int cw, int k, int8_t* dst,
                                              int8_t* Edst, int kid, long long idx0) {
    int v[32], e[32], q[32];
#pragma unroll
    for (int i = 0; i < 32; i++) {
        v[i] = (int)(int8_t)(tile[rb * 32 + i][cw] >> (8 * k));
        e[i] = et[rb * 32 + i][cw >> 3];
    }
    const int Eo = quant_geral<32, 1>(v, e, q, kid, idx0);
#pragma unroll
    for (int i4 = 0; i4 < 8; i4++) reinterpret_cast<uint32_t*>(dst)[i4] = junta4(q[4 * i4], q[4 * i4 + 1], q[4 * i4 + 2], q[4 * i4 + 3]);
    *Edst = (int8_t)Eo;
    return Eo;
}

// per-byte signed maximum into a 4-byte-aligned word of an int8 array
__device__ __forceinline__ void max4_atomico(int8_t* p, uint32_t meu) {
    unsigned* w = reinterpret_cast<unsigned*>(p);
    unsigned visto = *w;
    for (;;) {
        const unsigned novo = __vmaxs4(visto, meu);
        if (novo == visto) return;
        const unsigned antes = atomicCAS(w, visto, novo);
        if (antes == visto) return;
        visto = antes;
    }
}

template <int TR, int CPT>
__device__ __forceinline__ void transpoe32_corpo(const int8_t* __restrict__ X, const int8_t* __restrict__ EX, int8_t* __restrict__ Y,
                                                 int8_t* __restrict__ EY, int R, int C, int kid, int8_t* __restrict__ RM = nullptr) {
    pdl_espera();
    pdl_solta();
    static_assert(CPT == 4 || CPT == 1, "a thread owns the 4 columns of a word or one of them");
    constexpr int TC = 256, PW = T32_PW, NT = 8 * TR / CPT, NPAR = (TR / 32) * 8;
    __shared__ uint32_t tile[TR][PW];
    __shared__ __align__(4) int8_t et[TR][8];
    __shared__ float fA[TR][8];                   // 2^(e - largest exponent of the row's 32-row block), per 32-column block
    __shared__ int eref_s[NPAR];                  // that largest exponent; bit 30 set: exponents too far apart for fp32
    const int r0 = blockIdx.y * TR, c0 = blockIdx.x * TC;
    const int tid = threadIdx.x;
    const int nbx = C / 32, nby = R / 32;
#pragma unroll
    for (int k = 0; k < TR * 16 / NT; k++) {
        const int idx = tid + NT * k, lr = idx >> 4, c16 = idx & 15;
        const uint4 v = *reinterpret_cast<const uint4*>(X + (size_t)(r0 + lr) * C + c0 + c16 * 16);
        tile[lr][c16 * 4] = v.x; tile[lr][c16 * 4 + 1] = v.y; tile[lr][c16 * 4 + 2] = v.z; tile[lr][c16 * 4 + 3] = v.w;
    }
    if (tid < 2 * TR) {
        const int lr = tid >> 1, k4 = (tid & 1) * 4;
        *reinterpret_cast<uint32_t*>(&et[lr][k4]) = *reinterpret_cast<const uint32_t*>(EX + (size_t)(r0 + lr) * nbx + c0 / 32 + k4);
    }
    __syncthreads();
    // scales of the rows: a warp per (32-row block, 32-column block), a lane per row.  Rows of all-zero blocks do not count
    // for the spread (their mantissas are zero whatever the scale).
    for (int p = tid >> 5; p < NPAR; p += NT / 32) {
        const int rb = p >> 3, cb = p & 7, i = tid & 31;
        const int e = et[rb * 32 + i][cb];
        const int eref = __reduce_max_sync(0xffffffffu, e);
        const int emin = __reduce_min_sync(0xffffffffu, e == E_ZERO ? 127 : e);
        fA[rb * 32 + i][cb] = __int_as_float(max(127 + e - eref, 0) << 23);
        if (i == 0) eref_s[p] = (eref & 0xffff) | (eref - emin > 100 ? 1 << 30 : 0);
    }
    __syncthreads();
    // word column, 32-row block and (CPT = 1: small matrices, four times the threads) the byte of the word
    const int cw = tid & 63, rb = CPT == 4 ? tid >> 6 : tid >> 8, k_meu = (tid >> 6) & 3;
    const int er = eref_s[rb * 8 + (cw >> 3)];
    const int eref = (int)(int16_t)(er & 0xffff);
    const bool largo = (er >> 30) & 1;                              // spread too wide for the fp32 path
    const float* fa = &fA[rb * 32][cw >> 3];
    uint32_t emax4 = 0x80808080u;                                   // the new exponents of this thread's columns, -128 where it has none
#pragma unroll
    for (int k = 0; k < 4; k++) {
        if (CPT == 1 && k != k_meu) continue;
        const size_t col = (size_t)(c0 + 4 * cw + k);
        int8_t* dst = Y + col * R + r0 + rb * 32;
        int8_t* Edst = EY + col * nby + (r0 + rb * 32) / 32;
        if (largo) {
            const int Eo = transpoe32_lento(tile, et, rb, cw, k, dst, Edst, kid, (long long)col * R + r0 + rb * 32);
            emax4 = (emax4 & ~(0xffu << (8 * k))) | ((uint32_t)(uint8_t)(int8_t)Eo << (8 * k));
            continue;
        }
        float t[32], mx = 0.f;
#pragma unroll
        for (int i = 0; i < 32; i++) {
            t[i] = (float)(int)(int8_t)(tile[rb * 32 + i][cw] >> (8 * k)) * fa[8 * i];     // the words stay in shared memory: registers hold t
            mx = fmaxf(mx, fabsf(t[i]));
        }
        const int expo = (__float_as_int(mx) >> 23) - 127;          // floor(log2 mx); mx is a normal number or 0 here
        int Eo = eref + expo + 1 - 7;
        const bool morto = mx == 0.f || Eo < -126;
        if (!morto && Eo > 126) reporta(E_EXP, kid, (long long)col * R + r0 + rb * 32, Eo, eref);
        const float B = morto ? 0.f : __int_as_float((127 + 6 - expo) << 23);
        if (morto) Eo = E_ZERO;
        uint32_t saida[8];
#pragma unroll
        for (int i4 = 0; i4 < 8; i4++) {
            uint32_t r[4];
#pragma unroll
            for (int j = 0; j < 4; j++) r[j] = (uint32_t)__float_as_int(fmaf(t[4 * i4 + j], B, 12582912.0f));
            saida[i4] = __byte_perm(__byte_perm(r[0], r[1], 0x0040), __byte_perm(r[2], r[3], 0x0040), 0x5410);
        }
        reinterpret_cast<uint4*>(dst)[0] = make_uint4(saida[0], saida[1], saida[2], saida[3]);
        reinterpret_cast<uint4*>(dst)[1] = make_uint4(saida[4], saida[5], saida[6], saida[7]);
        *Edst = (int8_t)Eo;
        emax4 = (emax4 & ~(0xffu << (8 * k))) | ((uint32_t)(uint8_t)(int8_t)Eo << (8 * k));
    }
    // row maxima of the transposed tensor (what a GEMM aligns its rows to): the caller pre-set RM to -128
    if (RM != nullptr) max4_atomico(RM + c0 + 4 * cw, emax4);
}

template <int TR, int CPT = 4>
__global__ void __launch_bounds__(8 * TR / CPT, 768 / (8 * TR / CPT)) k_transpoe32(const int8_t* __restrict__ X, const int8_t* __restrict__ EX,
                                                                                   int8_t* __restrict__ Y, int8_t* __restrict__ EY, int R, int C,
                                                                                   int kid) {
    transpoe32_corpo<TR, CPT>(X, EX, Y, EY, R, C, kid);
}

// Two transpositions of matrices with the same number of rows in one launch (the two operands of a weight-gradient
// GEMM): blockIdx.z picks the matrix, the grid is as wide as the wider one.
struct ArgsTransp { const int8_t* X; const int8_t* EX; int8_t* Y; int8_t* EY; int C; int8_t* RM; };
template <int TR, int CPT = 4>
__global__ void __launch_bounds__(8 * TR / CPT, 768 / (8 * TR / CPT)) k_transpoe32_par(ArgsTransp a0, ArgsTransp a1, int R, int kid) {
    const ArgsTransp a = blockIdx.z ? a1 : a0;
    if ((int)blockIdx.x * 256 >= a.C) return;
    transpoe32_corpo<TR, CPT>(a.X, a.EX, a.Y, a.EY, R, a.C, kid, a.RM);
}

// RMSNorm without gain, one warp per row, NP*512 >= D columns held in registers.  ops.py:153-165
//   ss = sum_b rnd(sq_b << G, 2 (emax - e_b));  r = isqrt(ss >> log2D);  k = bitlen(r) + 10;  inv = 2^k / r
//   y = quant(x * inv, e_b - k - emax + G/2);  cache = (r, emax)
template <int BLK, int NP>
__global__ void __launch_bounds__(256) k_rms(const int8_t* __restrict__ Xm, const int8_t* __restrict__ XE, int8_t* __restrict__ Ym,
                                             int8_t* __restrict__ YE, int* __restrict__ cr, int* __restrict__ cemax, int M, int D, int log2D, int G,
                                             int kid) {
    pdl_espera();
    pdl_solta();
    constexpr int GL = BLK / 16;
    const int lane = threadIdx.x & 31;
    const long long lin_ = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
    const bool linha_ok = lin_ < M;
    const long long lin = linha_ok ? lin_ : 0;
    const int nb = D / BLK;
    int x[NP][16], eb[NP];
    bool tem[NP];
    int emax = -128;
#pragma unroll
    for (int p = 0; p < NP; p++) {
        const int c = (p * 32 + lane) * 16;
        tem[p] = c < D;
        if (tem[p]) {
            le16(Xm + lin * D + c, x[p]);
            eb[p] = XE[lin * nb + c / BLK];
            emax = max(emax, eb[p]);
        } else {
#pragma unroll
            for (int i = 0; i < 16; i++) x[p][i] = 0;
            eb[p] = E_ZERO;
        }
    }
    emax = warp_max(emax);
    int ss = 0;
#pragma unroll
    for (int p = 0; p < NP; p++) {
        int sq = 0;
#pragma unroll
        for (int i = 0; i < 16; i++) sq += x[p][i] * x[p][i];
#pragma unroll
        for (int o = GL / 2; o; o >>= 1) sq += __shfl_xor_sync(FULL, sq, o);      // whole block on every lane of the group
        if ((lane % GL) == 0 && tem[p]) ss += rnd_d(sq << G, 2 * (emax - eb[p]));
    }
    ss = warp_sum(ss);
    const int r = isqrt_i(ss >> log2D);
    const int k = bitlen(r) + 10;
    const int inv = (1 << k) / r;
    const float invf = (float)inv;                   // inv <= 2^11 and |x| <= 127: x * inv < 2^18 is exact in fp32
#pragma unroll
    for (int p = 0; p < NP; p++) {
        float f[16];
#pragma unroll
        for (int i = 0; i < 16; i++) f[i] = (float)x[p][i] * invf;
        const int c = (p * 32 + lane) * 16;
        uint4 pac;
        const int Eo = quant_f32<GL>(f, eb[p] - k - emax + G / 2, pac, kid, lin * D + c);
        if (tem[p] && linha_ok) {
            *reinterpret_cast<uint4*>(Ym + lin * D + c) = pac;
            if ((lane % GL) == 0) YE[lin * nb + c / BLK] = (int8_t)Eo;
        }
    }
    if (lane == 0 && linha_ok) { cr[lin] = r; cemax[lin] = emax; }
}

// RMSNorm backward: dx = (g - y * mean(g y)) / rms with two shrink steps (15 and 18 bits).  ops.py:167-184
// SOMA: the result is added to the block tensor x (the residual gradient) before it is stored: soma(x, rms_back(...)).
template <int BLK, int NP, bool SOMA>
__device__ __forceinline__ void rms_back_corpo(const int8_t* __restrict__ gm, const int8_t* __restrict__ gE, const int8_t* __restrict__ ym,
                                               const int8_t* __restrict__ yE, const int* __restrict__ cr, const int* __restrict__ cemax,
                                               const int8_t* __restrict__ xm, const int8_t* __restrict__ xE, int8_t* __restrict__ om,
                                               int8_t* __restrict__ oE, int M, int D, int log2D, int G, int GB, int kid) {
    pdl_espera();
    pdl_solta();
    constexpr int GL = BLK / 16;
    const int lane = threadIdx.x & 31;
    const long long lin_ = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
    const bool linha_ok = lin_ < M;
    const long long lin = linha_ok ? lin_ : 0;
    const int nb = D / BLK;
    int g[NP][16], y[NP][16], eg[NP], ey[NP];
    bool tem[NP];
    int smax = -100000;
#pragma unroll
    for (int p = 0; p < NP; p++) {
        const int c = (p * 32 + lane) * 16;
        tem[p] = c < D;
        if (tem[p]) {
            le16(gm + lin * D + c, g[p]);
            le16(ym + lin * D + c, y[p]);
            eg[p] = gE[lin * nb + c / BLK];
            ey[p] = yE[lin * nb + c / BLK];
            smax = max(smax, eg[p] + ey[p]);
        } else {
#pragma unroll
            for (int i = 0; i < 16; i++) g[p][i] = y[p][i] = 0;
            eg[p] = ey[p] = E_ZERO;
        }
    }
    smax = warp_max(smax);
    int S = 0;
#pragma unroll
    for (int p = 0; p < NP; p++) {
        const int s = smax - (eg[p] + ey[p]);
#pragma unroll
        for (int i = 0; i < 16; i++) S += rnd_d((g[p][i] * y[p][i]) << GB, s);
    }
    S = warp_sum(S);
    int eS = smax - GB - log2D;
    const int sh = max(bitlen(S) - 15, 0);
    S = rnd_d(S, sh);
    eS += sh;
    const int r = cr[lin], emax = cemax[lin];
    const int k = bitlen(r) + 10;
    const int inv = (1 << k) / max(r, 1);
#pragma unroll
    for (int p = 0; p < NP; p++) {
        const int c = (p * 32 + lane) * 16;
        const long long o = lin * D + c;
        const int ec = max(eg[p] + 7, ey[p] + eS + 22) - 28;
        int v[16], e[16], q[16];
#pragma unroll
        for (int i = 0; i < 16; i++) {
            // ec >= eg + 7 - 28 and ec >= ey + eS + 22 - 28: the 7-bit g moves up by at most 21, the 22-bit y S by at most 6
            int dentro = desloca(g[p][i], ec - eg[p]) - desloca(y[p][i] * S, ec - (ey[p] + eS));
            const int sh2 = max(bitlen(dentro) - 18, 0);
            dentro = rnd_d(dentro, sh2);
            v[i] = dentro * inv;
            e[i] = ec + sh2 - k - (emax - G / 2);
        }
        int Eo = quant_geral<16, GL>(v, e, q, kid, o);
        if (SOMA) {
            int xv[16];
            uint4 pac;
            if (tem[p]) le16(xm + o, xv);
            else {
#pragma unroll
                for (int i = 0; i < 16; i++) xv[i] = 0;
            }
            Eo = soma16<GL>(xv, tem[p] ? (int)xE[lin * nb + c / BLK] : E_ZERO, q, (int)(int8_t)Eo, pac, kid, o);
            if (tem[p] && linha_ok) *reinterpret_cast<uint4*>(om + o) = pac;
        } else if (tem[p] && linha_ok) grava16(om + o, q);
        if (tem[p] && linha_ok && (lane % GL) == 0) oE[lin * nb + c / BLK] = (int8_t)Eo;
    }
}
template <int BLK, int NP>
__global__ void __launch_bounds__(256) k_rms_back(const int8_t* __restrict__ gm, const int8_t* __restrict__ gE, const int8_t* __restrict__ ym,
                                                  const int8_t* __restrict__ yE, const int* __restrict__ cr, const int* __restrict__ cemax,
                                                  int8_t* __restrict__ om, int8_t* __restrict__ oE, int M, int D, int log2D, int G, int GB, int kid) {
    rms_back_corpo<BLK, NP, false>(gm, gE, ym, yE, cr, cemax, nullptr, nullptr, om, oE, M, D, log2D, G, GB, kid);
}
template <int BLK, int NP>
__global__ void __launch_bounds__(256) k_rms_back_soma(const int8_t* __restrict__ gm, const int8_t* __restrict__ gE, const int8_t* __restrict__ ym,
                                                       const int8_t* __restrict__ yE, const int* __restrict__ cr, const int* __restrict__ cemax,
                                                       const int8_t* __restrict__ xm, const int8_t* __restrict__ xE, int8_t* __restrict__ om,
                                                       int8_t* __restrict__ oE, int M, int D, int log2D, int G, int GB, int kid) {
    rms_back_corpo<BLK, NP, true>(gm, gE, ym, yE, cr, cemax, xm, xE, om, oE, M, D, log2D, G, GB, kid);
}

// integer softmax + cross-entropy gradient, one warp per row of raw logits.  ops.py:260-271
//   u = rnd(acc, -(e + 8)); ex = exp(-(umax - u)/256) >> 3; s = sum ex; v = (ex * (2^28 / s) + 2^15) >> 16;
//   v[target] -= 4096; g = quant(v, -12 - log2M); also d_alvo = umax - u[target] and s for the loss report.
template <int BLK, int NP>
__global__ void __launch_bounds__(256) k_softmax_ce(const int* __restrict__ acc, const int16_t* __restrict__ e, const int* __restrict__ alvo,
                                                    int8_t* __restrict__ gm, int8_t* __restrict__ gE, int* __restrict__ d_alvo, int* __restrict__ soma,
                                                    int M, int V, int log2M, int kid) {
    pdl_espera();
    pdl_solta();
    constexpr int GL = BLK / 16;
    const int lane = threadIdx.x & 31;
    const long long lin_ = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
    const bool linha_ok = lin_ < M;
    const long long lin = linha_ok ? lin_ : 0;
    int u[NP][16];
    bool tem[NP];
    int umax = U_MIN;
    const int tk = alvo[lin];
    if (lane == 0 && linha_ok && (tk < 0 || tk >= V)) reporta(E_ARG, kid, lin * V, tk, V);
#pragma unroll
    for (int p = 0; p < NP; p++) {
        const int c = (p * 32 + lane) * 16;
        tem[p] = c < V;
        if (tem[p]) {
            int a[16], ee[16];
            le16_i32(acc + lin * V + c, a);
            le16_i16(e + lin * V + c, ee);
#pragma unroll
            for (int i = 0; i < 16; i++) {
                u[p][i] = rnd(a[i], -(ee[i] + 8), kid, lin * V + c + i);
                umax = max(umax, u[p][i]);
            }
        } else {
#pragma unroll
            for (int i = 0; i < 16; i++) u[p][i] = U_MIN;
        }
    }
    umax = warp_max(umax);
    int s = 0, ut = U_MIN;
#pragma unroll
    for (int p = 0; p < NP; p++) {
        const int c = (p * 32 + lane) * 16;
#pragma unroll
        for (int i = 0; i < 16; i++) {
            if (c + i == tk) ut = u[p][i];
            u[p][i] = tem[p] ? exp_dif(umax, u[p][i]) >> 3 : 0;          // u now holds ex
            s += u[p][i];
        }
    }
    s = warp_sum(s);
    ut = warp_max(ut);
    if (s <= 0) { if (lane == 0 && linha_ok) reporta(E_DIV, kid, lin * V, s, 0); s = 1; }
    const int inv = (1 << 28) / s;
#pragma unroll
    for (int p = 0; p < NP; p++) {
        const int c = (p * 32 + lane) * 16;
        int v[16], q[16];
#pragma unroll
        for (int i = 0; i < 16; i++) v[i] = ((u[p][i] * inv + (1 << 15)) >> 16) - (c + i == tk ? 4096 : 0);
        const int Eo = quant_uniforme<16, GL>(v, -12 - log2M, q, kid, lin * V + c);
        if (tem[p] && linha_ok) {
            grava16(gm + lin * V + c, q);
            if ((lane % GL) == 0) gE[lin * (V / BLK) + c / BLK] = (int8_t)Eo;
        }
    }
    if (lane == 0 && linha_ok) { d_alvo[lin] = umax - ut; soma[lin] = s; }
}

}  // namespace jt
