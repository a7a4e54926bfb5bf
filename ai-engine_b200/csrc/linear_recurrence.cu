// Linear attention with a decaying matrix state, per request and head:
//     S_t = diag(a_t) S_(t-1) + k_t v_t^T        (S: [d, dv], a_t per key channel)
//     o_t = S_t^T q_t
// a_t is a constant per head (retention) or a per-token, per-channel value (gated linear attention).  The
// state is float32, lives in the request's slot and is carried from step to step.
//
// The columns of S never mix: column j needs only v_t[j].  A warp owns 32 / lanes columns of one (request,
// head); `lanes` threads share a column, each with RPT consecutive rows of S in registers, and a token costs
// each thread 2 RPT multiply-adds and a shuffle reduction over its column's lanes.  Tokens of a portion run
// in order, so a portion of any length continues where the previous step left the state, and a request's
// result does not depend on what else is in the batch.
#include "common.cuh"

template <int RPT>
__global__ void __launch_bounds__(128)
linear_recurrence_kernel(const float* __restrict__ q, const float* __restrict__ k, const float* __restrict__ v, int ld,
                         const float* __restrict__ decay_tok, int ld_decay, const float* __restrict__ decay_head,
                         float q_scale, float k_scale, float* __restrict__ state, float* __restrict__ out,
                         const int* __restrict__ q_start, const int* __restrict__ q_len, const int* __restrict__ slots,
                         int R, int H, int d, int dv, int lanes, int groups, int max_slots, int vec, unsigned* err) {
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (warp >= R * H * groups) return;
    const int cg = warp % groups, h = (warp / groups) % H, r = warp / (groups * H);
    const int slot = slots[r];
    if (slot < 0 || slot >= max_slots) {
        if (lane == 0) atomicOr(err, AIE_DEV_SLOT_OOB);
        return;
    }
    const int cols = 32 / lanes;
    const int g = lane % lanes, col = cg * cols + lane / lanes;
    const int row0 = g * RPT;
    const bool col_ok = col < dv;
    float S[RPT];
    float* sp = state + (((size_t)slot * H + h) * d) * dv + col;
#pragma unroll
    for (int i = 0; i < RPT; ++i) S[i] = (col_ok && row0 + i < d) ? sp[(size_t)(row0 + i) * dv] : 0.f;
    const float dh = decay_head ? decay_head[h] : 1.f;
    const int a = q_start[r], n = q_len[r];
    for (int t = a; t < a + n; ++t) {
        const float* qr = q + (size_t)t * ld + h * d + row0;
        const float* kr = k + (size_t)t * ld + h * d + row0;
        const float* ar = decay_tok ? decay_tok + (size_t)t * ld_decay + h * d + row0 : nullptr;
        const float vv = col_ok ? v[(size_t)t * ld + h * dv + col] * k_scale : 0.f;
        float o = 0.f;
        if (vec) {
#pragma unroll
            for (int i = 0; i < RPT; i += 4) {
                if (row0 + i < d) {
                    const float4 q4 = *reinterpret_cast<const float4*>(qr + i);
                    const float4 k4 = *reinterpret_cast<const float4*>(kr + i);
                    float4 a4 = make_float4(dh, dh, dh, dh);
                    if (ar) a4 = *reinterpret_cast<const float4*>(ar + i);
                    S[i] = fmaf(a4.x, S[i], k4.x * vv);
                    S[i + 1] = fmaf(a4.y, S[i + 1], k4.y * vv);
                    S[i + 2] = fmaf(a4.z, S[i + 2], k4.z * vv);
                    S[i + 3] = fmaf(a4.w, S[i + 3], k4.w * vv);
                    o = fmaf(S[i], q4.x, o);
                    o = fmaf(S[i + 1], q4.y, o);
                    o = fmaf(S[i + 2], q4.z, o);
                    o = fmaf(S[i + 3], q4.w, o);
                }
            }
        } else {
#pragma unroll
            for (int i = 0; i < RPT; ++i) {
                if (row0 + i < d) {
                    const float al = ar ? ar[i] : dh;
                    S[i] = fmaf(al, S[i], kr[i] * vv);
                    o = fmaf(S[i], qr[i], o);
                }
            }
        }
        for (int off = lanes >> 1; off > 0; off >>= 1) o += __shfl_xor_sync(0xffffffffu, o, off);
        if (g == 0 && col_ok) out[((size_t)t * H + h) * dv + col] = o * q_scale;
    }
    if (col_ok) {
#pragma unroll
        for (int i = 0; i < RPT; ++i)
            if (row0 + i < d) sp[(size_t)(row0 + i) * dv] = S[i];
    }
}

// q, k [T, .] with head h's d channels at column h d of rows `ld` floats apart; v likewise with dv columns a
// head; decay_tok [T, .] rows `ld_decay` apart (or null: decay_head [H] constants).  The key is scaled by
// k_scale, the output by q_scale (both 1 or d^-1/2).  state [max_slots, H, d, dv]; out [T, H, dv].
extern "C" int aie_linear_recurrence(const float* q, const float* k, const float* v, int ld, const float* decay_tok,
                                     int ld_decay, const float* decay_head, float q_scale, float k_scale, float* state,
                                     float* out, const int* q_start, const int* q_len, const int* slots, int R, int H,
                                     int d, int dv, int max_slots, unsigned* err, cudaStream_t st) {
    if (R <= 0) return 0;
    if (H <= 0 || d <= 0 || dv <= 0 || (!decay_tok && !decay_head)) return AIE_BAD_ARG;
    if (d > 1024) return AIE_UNSUPPORTED;
    const int rpt = d <= 32 ? 8 : (d <= 128 ? 16 : 32);
    int lanes = 1;
    while (lanes * rpt < d) lanes <<= 1;
    const int cols = 32 / lanes, groups = (dv + cols - 1) / cols;
    const long long warps = (long long)R * H * groups;
    const unsigned blocks = (unsigned)((warps + 3) / 4);
    const int vec = (d % 4 == 0 && ld % 4 == 0 && (!decay_tok || ld_decay % 4 == 0) && !((size_t)q & 15) &&
                     !((size_t)k & 15) && (!decay_tok || !((size_t)decay_tok & 15))) ? 1 : 0;
#define GO(N)                                                                                                       \
    linear_recurrence_kernel<N><<<blocks, 128, 0, st>>>(q, k, v, ld, decay_tok, ld_decay, decay_head, q_scale, k_scale, \
                                                        state, out, q_start, q_len, slots, R, H, d, dv, lanes, groups, \
                                                        max_slots, vec, err)
    if (rpt == 8) GO(8);
    else if (rpt == 16) GO(16);
    else GO(32);
#undef GO
    AIE_LAUNCH_CHECK();
}
