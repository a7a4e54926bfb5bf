// The scalar-decay state-space recurrence of a prompt portion in chunks, on tensor cores:
//     S_t = a_t S_(t-1) + dt_t B_t x_t^T,   y_t = S_t^T C_t + skip x_t      (S: [N, dv] per head, float32)
// with dt_t = softplus(raw_t + bias), a_t = exp(-exp(a_log) dt_t).  Token by token this is a chain of dependent
// rank-1 updates; over a chunk of Q tokens it is four matrix products.  With l_t = sum_{s <= t} log a_s (float32):
//     G = C B^T                                   [Q, Q]   which key meets which query
//     W[t, s] = G[t, s] exp(l_t - l_s) dt_s   (s <= t, else 0)
//     Y = W X + diag(exp(l_t)) (C S_prev)         [Q, dv]
//     S_new = exp(l_Q) S_prev + B^T (w * X),   w_s = exp(l_Q - l_s) dt_s
// One CTA owns a (request, head, 64 or 32 value columns) and walks the request's chunks in order with the state in shared
// memory, so a portion continues where the last step stopped and no result depends on the batch.  x, B and C (outputs
// of the convolution and its activation) enter the products rounded to bfloat16; everything that holds a decay, a
// step size or the state (W, w * X, S) enters as a pair of bfloat16 values, the rounded value and the rounded rest,
// which carries 16 bits of mantissa; sums are float32.  Exponents are never positive: nothing can overflow.
#include <mma.h>

#include "common.cuh"

using namespace nvcuda;

#define SC_Q 64
#define SC_THREADS 512
#define SC_PAD 8         // bfloat16 elements (16 bytes) behind every row in shared memory: rows of a tile fall into
#define SC_PADF 4        // different banks (the same 16 bytes for float32 rows)
#define SC_WARPS 16

typedef wmma::fragment<wmma::matrix_a, 16, 16, 16, bf16, wmma::row_major> FragA;
typedef wmma::fragment<wmma::matrix_a, 16, 16, 16, bf16, wmma::col_major> FragAT;
typedef wmma::fragment<wmma::matrix_b, 16, 16, 16, bf16, wmma::row_major> FragB;
typedef wmma::fragment<wmma::matrix_b, 16, 16, 16, bf16, wmma::col_major> FragBT;
typedef wmma::fragment<wmma::accumulator, 16, 16, 16, float> FragC;

__device__ __forceinline__ void split_bf16(float v, bf16* hi, bf16* lo) {
    const bf16 h = __float2bfloat16_rn(v);
    *hi = h;
    *lo = __float2bfloat16_rn(v - __bfloat162float(h));
}

// NP: the state's rows padded to a multiple of 16 (zero rows and columns change nothing); DV: value columns a CTA
template <int NP, int DV>
__global__ void __launch_bounds__(SC_THREADS)
state_space_chunked_kernel(const float* __restrict__ Cg, const float* __restrict__ Bg, const float* __restrict__ Xg, int ld,
                           const float* __restrict__ dt_raw, int ld_dt, const float* __restrict__ dt_bias,
                           const float* __restrict__ a_log, const float* __restrict__ skip, float* __restrict__ state,
                           float* __restrict__ out, const int* __restrict__ q_start, const int* __restrict__ q_len,
                           const int* __restrict__ slots, int H, int N, int dv, int hpg, int col_blocks, int max_slots,
                           int min_len, unsigned* err) {
    extern __shared__ __align__(128) unsigned char sc_sm[];
    const int tid = threadIdx.x, warp = tid >> 5;
    const int cb = blockIdx.x % col_blocks, h = (blockIdx.x / col_blocks) % H, r = blockIdx.x / (col_blocks * H);
    const int n_tok = q_len[r];
    if (n_tok < min_len) return;                       // short portions and single tokens take the token-by-token kernel
    const int slot = slots[r];
    if (slot < 0 || slot >= max_slots) {
        if (tid == 0) atomicOr(err, AIE_DEV_SLOT_OOB);
        return;
    }
    constexpr int LN = NP + SC_PAD, LD = DV + SC_PAD, LQ = SC_Q + SC_PAD;      // row strides, bfloat16 buffers
    constexpr int FQ = SC_Q + SC_PADF, FD = DV + SC_PADF;                      // ... float32 buffers
    constexpr int FY = FQ > FD ? FQ : FD;                                      // G and Ya share a place
    constexpr int DT = DV / 16;                                                // column tiles of a CTA
    bf16* Cs = reinterpret_cast<bf16*>(sc_sm);                    // [Q][NP]
    bf16* Bs = Cs + SC_Q * LN;                                    // [Q][NP]
    bf16* XwH = Bs + SC_Q * LN;                                   // [Q][DV]  w * X, rounded
    bf16* XwL = XwH + SC_Q * LD;                                  //          ... and the rest
    bf16* Xs = XwL + SC_Q * LD;                                   // [Q][DV]
    bf16* WH = Xs + SC_Q * LD;                                    // [Q][Q]
    bf16* WL = WH + SC_Q * LQ;
    bf16* SH = WL + SC_Q * LQ;                                    // [NP][DV]
    bf16* SL = SH + NP * LD;
    float* Gf = reinterpret_cast<float*>(SL + NP * LD);           // [Q][Q], then Ya [Q][DV]
    float* Yb = Gf + SC_Q * FY;                                   // [Q][DV]
    float* Sf = Yb + SC_Q * FD;                                   // [NP][DV]
    float* la = Sf + NP * FD;                                     // [Q] running sums of log decays
    float* dtv = la + SC_Q;                                       // [Q] step sizes
    float* wv = dtv + SC_Q;                                       // [Q] w_s = exp(l_Q - l_s) dt_s
    float* ela = wv + SC_Q;                                       // [Q] exp(l_t)

    const int hq = h / hpg, col0 = cb * DV, a0 = q_start[r];
    const float rate = expf(a_log[h]), dtb = dt_bias[h], sk = skip ? skip[h] : 0.f;
    float* sp = state + ((size_t)slot * H + h) * N * dv;
    for (int i = tid; i < NP * DV; i += SC_THREADS) {
        const int n = i / DV, j = i % DV;
        const float v = (n < N && col0 + j < dv) ? sp[(size_t)n * dv + col0 + j] : 0.f;
        Sf[n * FD + j] = v;
        split_bf16(v, SH + n * LD + j, SL + n * LD + j);
    }
    for (int t0 = 0; t0 < n_tok; t0 += SC_Q) {
        const int nt = min(SC_Q, n_tok - t0);
        __syncthreads();                               // the last chunk is done with; the state's halves are written
        // the chunk's rows: fixed trip counts, unrolled, so that a thread's loads are all in flight before the first
        // is converted (the latency of memory is paid once a chunk, not once a row)
        {
            constexpr int PER = SC_Q * NP / SC_THREADS;
            float cv[PER], bv[PER];
#pragma unroll
            for (int it = 0; it < PER; ++it) {
                const int i = tid + it * SC_THREADS, t = i / NP, n = i % NP;
                const bool ok = t < nt && n < N;
                const size_t at = (size_t)(a0 + t0 + t) * ld + (size_t)hq * N + n;
                cv[it] = ok ? Cg[at] : 0.f;
                bv[it] = ok ? Bg[at] : 0.f;
            }
            constexpr int PERX = SC_Q * DV / SC_THREADS;
            float xv[PERX];
#pragma unroll
            for (int it = 0; it < PERX; ++it) {
                const int i = tid + it * SC_THREADS, t = i / DV, j = i % DV;
                xv[it] = (t < nt && col0 + j < dv) ? Xg[(size_t)(a0 + t0 + t) * ld + (size_t)h * dv + col0 + j] : 0.f;
            }
#pragma unroll
            for (int it = 0; it < PER; ++it) {
                const int i = tid + it * SC_THREADS, t = i / NP, n = i % NP;
                Cs[t * LN + n] = __float2bfloat16_rn(cv[it]);
                Bs[t * LN + n] = __float2bfloat16_rn(bv[it]);
            }
#pragma unroll
            for (int it = 0; it < PERX; ++it) {
                const int i = tid + it * SC_THREADS, t = i / DV, j = i % DV;
                Xs[t * LD + j] = __float2bfloat16_rn(xv[it]);
            }
        }
        if (tid < SC_Q) {
            float d = 0.f;
            if (tid < nt) {
                const float x = dt_raw[(size_t)(a0 + t0 + tid) * ld_dt + h] + dtb;
                d = x > 20.f ? x : log1pf(expf(x));
            }
            dtv[tid] = d;                              // a token behind the portion's end: no step, no decay
        }
        __syncthreads();
        if (warp == 0) {                               // running sums of the 64 log decays: a scan over pairs
            const int lane = tid & 31;
            const float v0 = -rate * dtv[2 * lane], v1 = -rate * dtv[2 * lane + 1];
            float run = v0 + v1;
            for (int o = 1; o < 32; o <<= 1) {
                const float up = __shfl_up_sync(0xffffffffu, run, o);
                if (lane >= o) run += up;
            }
            la[2 * lane] = run - v1;
            la[2 * lane + 1] = run;
            const float end = __shfl_sync(0xffffffffu, run, 31);
            wv[2 * lane] = expf(end - (run - v1)) * dtv[2 * lane];
            wv[2 * lane + 1] = expf(end - run) * dtv[2 * lane + 1];
            ela[2 * lane] = expf(run - v1);
            ela[2 * lane + 1] = expf(run);
        }
        // G = C B^T, the tiles on and below the diagonal
        for (int tile = warp; tile < 16; tile += SC_WARPS) {
            const int ti = tile >> 2, tj = tile & 3;
            if (tj > ti) continue;
            FragC acc;
            wmma::fill_fragment(acc, 0.f);
            for (int k = 0; k < NP / 16; ++k) {
                FragA fa;
                FragBT fb;
                wmma::load_matrix_sync(fa, Cs + ti * 16 * LN + k * 16, LN);
                wmma::load_matrix_sync(fb, Bs + tj * 16 * LN + k * 16, LN);
                wmma::mma_sync(acc, fa, fb, acc);
            }
            wmma::store_matrix_sync(Gf + ti * 16 * FY + tj * 16, acc, FY, wmma::mem_row_major);
        }
        __syncthreads();
        const float l_end = la[SC_Q - 1];
        // W on and below the diagonal, tile by tile (the tiles above it are never read)
        for (int i = tid; i < 10 * 256; i += SC_THREADS) {
            const int tile = i >> 8, e = i & 255;
            const int ti = tile < 1 ? 0 : (tile < 3 ? 1 : (tile < 6 ? 2 : 3)), tj = tile - ti * (ti + 1) / 2;
            const int t = ti * 16 + (e >> 4), s = tj * 16 + (e & 15);
            const float w = s <= t ? Gf[t * FY + s] * __expf(la[t] - la[s]) * dtv[s] : 0.f;
            split_bf16(w, WH + t * LQ + s, WL + t * LQ + s);
        }
        for (int i = tid; i < SC_Q * DV; i += SC_THREADS) {
            const int s = i / DV, j = i % DV;
            split_bf16(__bfloat162float(Xs[s * LD + j]) * wv[s], XwH + s * LD + j, XwL + s * LD + j);
        }
        __syncthreads();
        // Ya = W X (into G's place) and Yb = C S_prev
        for (int tile = warp; tile < 4 * DT; tile += SC_WARPS) {
            const int ti = tile / DT, tj = tile % DT;
            FragC acc;
            wmma::fill_fragment(acc, 0.f);
            for (int k = 0; k <= ti; ++k) {
                FragA fa;
                FragB fb;
                wmma::load_matrix_sync(fb, Xs + k * 16 * LD + tj * 16, LD);
                wmma::load_matrix_sync(fa, WH + ti * 16 * LQ + k * 16, LQ);
                wmma::mma_sync(acc, fa, fb, acc);
                wmma::load_matrix_sync(fa, WL + ti * 16 * LQ + k * 16, LQ);
                wmma::mma_sync(acc, fa, fb, acc);
            }
            wmma::store_matrix_sync(Gf + ti * 16 * FY + tj * 16, acc, FY, wmma::mem_row_major);
            wmma::fill_fragment(acc, 0.f);
            for (int k = 0; k < NP / 16; ++k) {
                FragA fa;
                FragB fb;
                wmma::load_matrix_sync(fa, Cs + ti * 16 * LN + k * 16, LN);
                wmma::load_matrix_sync(fb, SH + k * 16 * LD + tj * 16, LD);
                wmma::mma_sync(acc, fa, fb, acc);
                wmma::load_matrix_sync(fb, SL + k * 16 * LD + tj * 16, LD);
                wmma::mma_sync(acc, fa, fb, acc);
            }
            wmma::store_matrix_sync(Yb + ti * 16 * FD + tj * 16, acc, FD, wmma::mem_row_major);
        }
        // S = exp(l_end) S + B^T (w * X); a tile of the state belongs to one warp
        const float dec = expf(l_end);
        for (int tile = warp; tile < (NP / 16) * DT; tile += SC_WARPS) {
            const int ni = tile / DT, tj = tile % DT;
            FragC acc;
            wmma::load_matrix_sync(acc, Sf + ni * 16 * FD + tj * 16, FD, wmma::mem_row_major);
            for (int e = 0; e < acc.num_elements; ++e) acc.x[e] *= dec;
            for (int k = 0; k < SC_Q / 16; ++k) {
                FragAT fa;
                FragB fb;
                wmma::load_matrix_sync(fa, Bs + k * 16 * LN + ni * 16, LN);
                wmma::load_matrix_sync(fb, XwH + k * 16 * LD + tj * 16, LD);
                wmma::mma_sync(acc, fa, fb, acc);
                wmma::load_matrix_sync(fb, XwL + k * 16 * LD + tj * 16, LD);
                wmma::mma_sync(acc, fa, fb, acc);
            }
            wmma::store_matrix_sync(Sf + ni * 16 * FD + tj * 16, acc, FD, wmma::mem_row_major);
        }
        __syncthreads();
        for (int i = tid; i < SC_Q * DV; i += SC_THREADS) {
            const int t = i / DV, j = i % DV;
            if (t < nt && col0 + j < dv) {
                float y = fmaf(ela[t], Yb[t * FD + j], Gf[t * FY + j]);
                if (skip) y = fmaf(sk, __bfloat162float(Xs[t * LD + j]), y);      // x as the products saw it
                out[((size_t)(a0 + t0 + t) * H + h) * dv + col0 + j] = y;
            }
        }
        for (int i = tid; i < NP * DV; i += SC_THREADS) {
            const int n = i / DV, j = i % DV;
            split_bf16(Sf[n * FD + j], SH + n * LD + j, SL + n * LD + j);
        }
    }
    __syncthreads();
    for (int i = tid; i < NP * DV; i += SC_THREADS) {
        const int n = i / DV, j = i % DV;
        if (n < N && col0 + j < dv) sp[(size_t)n * dv + col0 + j] = Sf[n * FD + j];
    }
}

template <int NP, int DV> static size_t sc_smem() {
    const int LN = NP + SC_PAD, LD = DV + SC_PAD, LQ = SC_Q + SC_PAD, FQ = SC_Q + SC_PADF, FD = DV + SC_PADF;
    const int FY = FQ > FD ? FQ : FD;
    return (size_t)(2 * SC_Q * LN + 3 * SC_Q * LD + 2 * SC_Q * LQ + 2 * NP * LD) * sizeof(bf16) +
           (size_t)(SC_Q * FY + SC_Q * FD + NP * FD + 4 * SC_Q) * sizeof(float);
}

// C, B [T, .] with head h's N channels at column (h / hpg) N of rows `ld` floats apart; X likewise with dv columns a
// head at column h dv; dt_raw [T, .] rows ld_dt apart; state [max_slots, H, N, dv]; out [T, H, dv].  Requests that
// bring fewer than min_len tokens are left alone.  N <= 128.
extern "C" int aie_state_space_chunked(const float* C, const float* B, const float* X, int ld, const float* dt_raw, int ld_dt,
                                       const float* dt_bias, const float* a_log, const float* skip, float* state, float* out,
                                       const int* q_start, const int* q_len, const int* slots, int R, int H, int N, int dv,
                                       int hpg, int max_slots, int min_len, unsigned* err, cudaStream_t st) {
    if (R <= 0) return 0;
    if (H <= 0 || N <= 0 || dv <= 0 || hpg < 1 || H % hpg || !dt_raw || !dt_bias || !a_log) return AIE_BAD_ARG;
    if (N > 128) return AIE_UNSUPPORTED;
    // 64 value columns a CTA; 32 when that leaves SMs without one
    const bool narrow = dv > 32 && (long long)R * H * ((dv + 63) / 64) < aie_sm_count();
    const int DVc = narrow ? 32 : 64, col_blocks = (dv + DVc - 1) / DVc;
    const long long blocks = (long long)R * H * col_blocks;
    if (blocks > 0x7fffffffLL) return AIE_UNSUPPORTED;
#define GO(NP, DV)                                                                                                      \
    do {                                                                                                                \
        static bool set = false;                                                                                        \
        if (!set) {                                                                                                     \
            cudaError_t e = cudaFuncSetAttribute(state_space_chunked_kernel<NP, DV>,                                    \
                                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sc_smem<NP, DV>());  \
            if (e != cudaSuccess) return (int)e;                                                                        \
            set = true;                                                                                                 \
        }                                                                                                               \
        state_space_chunked_kernel<NP, DV><<<(unsigned)blocks, SC_THREADS, sc_smem<NP, DV>(), st>>>(                    \
            C, B, X, ld, dt_raw, ld_dt, dt_bias, a_log, skip, state, out, q_start, q_len, slots, H, N, dv, hpg, col_blocks, \
            max_slots, min_len, err);                                                                                   \
    } while (0)
#define GO2(NP)            \
    do {                   \
        if (narrow)        \
            GO(NP, 32);    \
        else               \
            GO(NP, 64);    \
    } while (0)
    if (N <= 16) GO2(16);
    else if (N <= 32) GO2(32);
    else if (N <= 64) GO2(64);
    else GO2(128);
#undef GO2
#undef GO
    AIE_LAUNCH_CHECK();
}
