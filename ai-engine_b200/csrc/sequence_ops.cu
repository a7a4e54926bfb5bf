// Row kernels of layers that carry more than a residual stream: a short causal convolution over time with
// its per-request tail, the weighted average over the streams of all earlier layers, activations that
// normalise over the feed-forward width or clamp their operands, a per-head norm with an output gate,
// per-channel decays from logits, and the bookkeeping of a mixture of experts whose experts are chosen
// by a table (rows grouped by expert, outputs summed per token).  Statistics, decays and sums are float32.
#include "common.cuh"

// ---------------------------------------------------------------------------
// out[t] = h[t] + sum_j w[:, j] * h[t - (taps-1) + j]      (per channel, zeros before the sequence's start)
// The inputs of the taps-1 tokens before a portion are the request's tail `state[slot]` [taps-1, D], oldest
// first.  Only the block of a request's first token of the step reads the tail: it computes the (at most
// taps-1) tokens that need it and then stores the new tail, so no other block races with the update.
// ---------------------------------------------------------------------------
template <typename O>
__global__ void short_conv_kernel(const float* __restrict__ h, const float* __restrict__ w, float* __restrict__ state,
                                  O* __restrict__ out, const int* __restrict__ q_start, const int* __restrict__ q_len,
                                  const int* __restrict__ slots, const int* __restrict__ token_req, int D, int taps,
                                  int max_slots, unsigned* err) {
    const int t = blockIdx.x, c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= D) return;
    const int r = token_req[t];
    const int a = q_start[r], n = q_len[r], i = t - a, slot = slots[r];
    const int Hh = taps - 1;
    const float* wc = w + (size_t)c * taps;
    if (i >= Hh) {
        float acc = h[(size_t)t * D + c];
        for (int j = 0; j < taps; ++j) acc = fmaf(wc[j], h[(size_t)(t - Hh + j) * D + c], acc);
        out[(size_t)t * D + c] = from_f32<O>(acc);
        return;
    }
    if (i != 0) return;
    if (slot < 0 || slot >= max_slots) {
        if (threadIdx.x == 0) atomicOr(err, AIE_DEV_SLOT_OOB);
        return;
    }
    float* st = state + (size_t)slot * Hh * D + c;          // st[k * D]: input at local index k - Hh
    const int first = min(n, Hh);
    for (int ii = 0; ii < first; ++ii) {
        float acc = h[(size_t)(a + ii) * D + c];
        for (int j = 0; j < taps; ++j) {
            const int src = ii - Hh + j;
            const float x = src >= 0 ? h[(size_t)(a + src) * D + c] : st[(size_t)(src + Hh) * D];
            acc = fmaf(wc[j], x, acc);
        }
        out[(size_t)(a + ii) * D + c] = from_f32<O>(acc);
    }
    for (int k = 0; k < Hh; ++k) {                          // ascending: entry n + k > k is still the old one
        const int src = n - Hh + k;
        st[(size_t)k * D] = src >= 0 ? h[(size_t)(a + src) * D + c] : st[(size_t)(n + k) * D];
    }
}

// The same for widths that are multiples of 4: a thread owns four neighbouring channels (16-byte loads).
template <typename O>
__global__ void short_conv4_kernel(const float* __restrict__ h, const float* __restrict__ w, float* __restrict__ state,
                                   O* __restrict__ out, const int* __restrict__ q_start, const int* __restrict__ q_len,
                                   const int* __restrict__ slots, const int* __restrict__ token_req, int D, int taps,
                                   int max_slots, unsigned* err) {
    const int t = blockIdx.x, c = (blockIdx.y * blockDim.x + threadIdx.x) * 4;
    if (c >= D) return;
    const int r = token_req[t];
    const int a = q_start[r], n = q_len[r], i = t - a, slot = slots[r];
    const int Hh = taps - 1;
    const float* wc = w + (size_t)c * taps;                 // channel c + e: wc[e * taps + j]
    if (i >= Hh) {
        float4 acc = *reinterpret_cast<const float4*>(h + (size_t)t * D + c);
        for (int j = 0; j < taps; ++j) {
            const float4 x = *reinterpret_cast<const float4*>(h + (size_t)(t - Hh + j) * D + c);
            acc.x = fmaf(wc[j], x.x, acc.x);
            acc.y = fmaf(wc[taps + j], x.y, acc.y);
            acc.z = fmaf(wc[2 * taps + j], x.z, acc.z);
            acc.w = fmaf(wc[3 * taps + j], x.w, acc.w);
        }
        store4<O>(out + (size_t)t * D + c, acc);
        return;
    }
    if (i != 0) return;
    if (slot < 0 || slot >= max_slots) {
        if (threadIdx.x == 0) atomicOr(err, AIE_DEV_SLOT_OOB);
        return;
    }
    float* st = state + (size_t)slot * Hh * D + c;
    const int first = min(n, Hh);
    for (int ii = 0; ii < first; ++ii) {
        float4 acc = *reinterpret_cast<const float4*>(h + (size_t)(a + ii) * D + c);
        for (int j = 0; j < taps; ++j) {
            const int src = ii - Hh + j;
            const float4 x = src >= 0 ? *reinterpret_cast<const float4*>(h + (size_t)(a + src) * D + c)
                                      : *reinterpret_cast<const float4*>(st + (size_t)(src + Hh) * D);
            acc.x = fmaf(wc[j], x.x, acc.x);
            acc.y = fmaf(wc[taps + j], x.y, acc.y);
            acc.z = fmaf(wc[2 * taps + j], x.z, acc.z);
            acc.w = fmaf(wc[3 * taps + j], x.w, acc.w);
        }
        store4<O>(out + (size_t)(a + ii) * D + c, acc);
    }
    for (int k = 0; k < Hh; ++k) {
        const int src = n - Hh + k;
        *reinterpret_cast<float4*>(st + (size_t)k * D) =
            src >= 0 ? *reinterpret_cast<const float4*>(h + (size_t)(a + src) * D + c)
                     : *reinterpret_cast<const float4*>(st + (size_t)(n + k) * D);
    }
}

extern "C" int aie_short_conv(const float* h, const float* w, float* state, void* out, int out_dtype, const int* q_start,
                              const int* q_len, const int* slots, const int* token_req, int T, int D, int taps,
                              int max_slots, unsigned* err, cudaStream_t st) {
    if (T <= 0) return 0;
    if (D <= 0 || taps < 1) return AIE_BAD_ARG;
    if (D % 4 == 0 && !((size_t)h & 15) && !((size_t)state & 15) && !((size_t)out & 15)) {
        const int threads = 64;
        dim3 grid4(T, (D / 4 + threads - 1) / threads);
        if (out_dtype == AIE_F32)
            short_conv4_kernel<float><<<grid4, threads, 0, st>>>(h, w, state, (float*)out, q_start, q_len, slots, token_req, D, taps, max_slots, err);
        else if (out_dtype == AIE_BF16)
            short_conv4_kernel<bf16><<<grid4, threads, 0, st>>>(h, w, state, (bf16*)out, q_start, q_len, slots, token_req, D, taps, max_slots, err);
        else
            return AIE_BAD_ARG;
        AIE_LAUNCH_CHECK();
    }
    dim3 grid(T, (D + 255) / 256);
    if (grid.y > 65535) return AIE_UNSUPPORTED;
    if (out_dtype == AIE_F32)
        short_conv_kernel<float><<<grid, 256, 0, st>>>(h, w, state, (float*)out, q_start, q_len, slots, token_req, D, taps, max_slots, err);
    else if (out_dtype == AIE_BF16)
        short_conv_kernel<bf16><<<grid, 256, 0, st>>>(h, w, state, (bf16*)out, q_start, q_len, slots, token_req, D, taps, max_slots, err);
    else
        return AIE_BAD_ARG;
    AIE_LAUNCH_CHECK();
}

// ---------------------------------------------------------------------------
// The stream that leaves layer i is a weighted sum of the streams all layers so far produced:
//   X = x (+ delta parts);  history[depth] = X;  x = sum_{j <= depth} coef[j] * history[j]
// history: [levels, n] float32 with n = T * D; x: [n] float32, rewritten in place.
// ---------------------------------------------------------------------------
template <typename A>
__global__ void depth_average_kernel(float* __restrict__ x, const A* __restrict__ delta, int parts, size_t part_stride,
                                     float* __restrict__ history, const float* __restrict__ coef, int depth, size_t n) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    float s = x[i];
    for (int p = 0; p < parts; ++p) s += to_f32<A>(delta[p * part_stride + i]);
    history[(size_t)depth * n + i] = s;
    float acc = 0.f;
    for (int j = 0; j < depth; ++j) acc = fmaf(coef[j], history[(size_t)j * n + i], acc);
    x[i] = fmaf(coef[depth], s, acc);
}

extern "C" int aie_depth_average(float* x, const void* delta, int delta_dtype, int parts, long long part_stride,
                                 float* history, const float* coef, int depth, long long n, cudaStream_t st) {
    if (n <= 0) return 0;
    if (depth < 0) return AIE_BAD_ARG;
    const unsigned blocks = (unsigned)((n + 255) / 256);
    if (!delta) parts = 0;
    if (delta_dtype == AIE_BF16 && delta)
        depth_average_kernel<bf16><<<blocks, 256, 0, st>>>(x, (const bf16*)delta, parts, (size_t)part_stride, history, coef, depth, (size_t)n);
    else
        depth_average_kernel<float><<<blocks, 256, 0, st>>>(x, (const float*)delta, parts, (size_t)part_stride, history, coef, depth, (size_t)n);
    AIE_LAUNCH_CHECK();
}

// ---------------------------------------------------------------------------
// A polynomial of normalised powers over the feed-forward width F, per token:
//   out = a N(z) + b N(z^2) + c N(z^3) + e,   N(y) = y / sqrt(mean(y^2) + eps)
// ---------------------------------------------------------------------------
template <typename O>
__global__ void polynorm_kernel(const float* __restrict__ z, const float* __restrict__ coef, O* __restrict__ out, int F,
                                float eps) {
    __shared__ float red[32];
    const float* zr = z + (size_t)blockIdx.x * F;
    float s2 = 0.f, s4 = 0.f, s6 = 0.f;
    for (int i = threadIdx.x; i < F; i += blockDim.x) {
        const float v = zr[i], v2 = v * v, v3 = v2 * v;
        s2 += v2;
        s4 += v2 * v2;
        s6 += v3 * v3;
    }
    s2 = block_sum(s2, red);
    s4 = block_sum(s4, red);
    s6 = block_sum(s6, red);
    const float r1 = 1.0f / sqrtf(s2 / (float)F + eps), r2 = 1.0f / sqrtf(s4 / (float)F + eps),
                r3 = 1.0f / sqrtf(s6 / (float)F + eps);
    const float a = coef[0] * r1, b = coef[1] * r2, c = coef[2] * r3, e = coef[3];
    for (int i = threadIdx.x; i < F; i += blockDim.x) {
        const float v = zr[i], v2 = v * v;
        out[(size_t)blockIdx.x * F + i] = from_f32<O>(a * v + b * v2 + c * (v2 * v) + e);
    }
}

extern "C" int aie_polynorm(const float* z, const float* coef, void* out, int out_dtype, int T, int F, float eps,
                            cudaStream_t st) {
    if (T <= 0) return 0;
    if (F <= 0) return AIE_BAD_ARG;
    const int threads = F >= 2048 ? 512 : 256;
    if (out_dtype == AIE_F32)
        polynorm_kernel<float><<<T, threads, 0, st>>>(z, coef, (float*)out, F, eps);
    else if (out_dtype == AIE_BF16)
        polynorm_kernel<bf16><<<T, threads, 0, st>>>(z, coef, (bf16*)out, F, eps);
    else
        return AIE_BAD_ARG;
    AIE_LAUNCH_CHECK();
}

// ---------------------------------------------------------------------------
// Per (token, head): y = o / sqrt(mean(o^2) + eps) (* w) * silu(g).  o [T, H, dv] float32; g has rows of
// `ldg` floats (a slice of a wider projection); w [dv] or null.  One warp per (token, head).
// ---------------------------------------------------------------------------
template <typename O>
__global__ void head_norm_gate_kernel(const float* __restrict__ o, const float* __restrict__ g, int ldg,
                                      const float* __restrict__ w, O* __restrict__ out, int TH, int H, int dv, float eps) {
    const int wi = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (wi >= TH) return;
    const int t = wi / H, hh = wi % H;
    const float* orow = o + (size_t)wi * dv;
    float ss = 0.f;
    for (int i = lane; i < dv; i += 32) ss += orow[i] * orow[i];
    ss = warp_sum(ss);
    const float r = 1.0f / sqrtf(ss / (float)dv + eps);
    const float* grow = g + (size_t)t * ldg + (size_t)hh * dv;
    for (int i = lane; i < dv; i += 32) {
        const float gv = grow[i];
        float y = orow[i] * r;
        if (w) y *= w[i];
        out[(size_t)wi * dv + i] = from_f32<O>(y * (gv / (1.0f + expf(-gv))));
    }
}

extern "C" int aie_head_norm_gate(const float* o, const float* g, int ldg, const float* w, void* out, int out_dtype, int T,
                                  int H, int dv, float eps, cudaStream_t st) {
    if (T <= 0) return 0;
    if (H <= 0 || dv <= 0) return AIE_BAD_ARG;
    const long long warps = (long long)T * H;
    const unsigned blocks = (unsigned)((warps + 3) / 4);
    if (out_dtype == AIE_F32)
        head_norm_gate_kernel<float><<<blocks, 128, 0, st>>>(o, g, ldg, w, (float*)out, (int)warps, H, dv, eps);
    else if (out_dtype == AIE_BF16)
        head_norm_gate_kernel<bf16><<<blocks, 128, 0, st>>>(o, g, ldg, w, (bf16*)out, (int)warps, H, dv, eps);
    else
        return AIE_BAD_ARG;
    AIE_LAUNCH_CHECK();
}

// ---------------------------------------------------------------------------
// A gated unit whose operands are clamped: g = min(gate, limit), u = clamp(up, -limit, limit),
//   y = g * sigmoid(alpha g) * (u + shift).   gu rows of `ld` floats: gate in [0, F), up in [F, 2F).
// ---------------------------------------------------------------------------
template <typename O>
__global__ void clamped_glu_kernel(const float* __restrict__ gu, int ld, O* __restrict__ out, long long n, int F,
                                   float limit, float alpha, float shift) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const long long t = i / F;
    const int f = (int)(i % F);
    const float g = fminf(gu[t * ld + f], limit);
    const float u = fminf(fmaxf(gu[t * ld + F + f], -limit), limit);
    out[i] = from_f32<O>(g / (1.0f + expf(-alpha * g)) * (u + shift));
}

extern "C" int aie_clamped_glu(const float* gu, int ld, void* out, int out_dtype, long long T, int F, float limit,
                               float alpha, float shift, cudaStream_t st) {
    if (T <= 0) return 0;
    if (F <= 0) return AIE_BAD_ARG;
    const long long n = T * F;
    const unsigned blocks = (unsigned)((n + 255) / 256);
    if (out_dtype == AIE_F32)
        clamped_glu_kernel<float><<<blocks, 256, 0, st>>>(gu, ld, (float*)out, n, F, limit, alpha, shift);
    else if (out_dtype == AIE_BF16)
        clamped_glu_kernel<bf16><<<blocks, 256, 0, st>>>(gu, ld, (bf16*)out, n, F, limit, alpha, shift);
    else
        return AIE_BAD_ARG;
    AIE_LAUNCH_CHECK();
}

// ---------------------------------------------------------------------------
// decay = sigmoid(z + bias)^(1 / tau) = exp(log_sigmoid(z + bias) / tau), float32 throughout.
// ---------------------------------------------------------------------------
__global__ void gated_decay_kernel(const float* __restrict__ z, const float* __restrict__ bias, float* __restrict__ out,
                                   long long n, int N, float inv_tau) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const float v = z[i] + (bias ? bias[i % N] : 0.f);
    const float ls = fminf(v, 0.f) - log1pf(expf(-fabsf(v)));      // log(sigmoid(v)), stable on both sides
    out[i] = expf(ls * inv_tau);
}

extern "C" int aie_gated_decay(const float* z, const float* bias, float* out, long long T, int N, float tau,
                               cudaStream_t st) {
    if (T <= 0) return 0;
    if (N <= 0 || !(tau > 0.f)) return AIE_BAD_ARG;
    const long long n = T * N;
    gated_decay_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(z, bias, out, n, N, 1.0f / tau);
    AIE_LAUNCH_CHECK();
}

// ---------------------------------------------------------------------------
// Experts chosen by a table of the token's id: pair p = (token t, choice s) goes to expert table[id[t], s].
// One block groups the pairs by expert into tiles of `tile` rows (each expert's rows padded up to whole tiles):
//   row_token[row]  = token of the row, -1 for padding         [n_tiles * tile]
//   pair_row[p]     = row of pair p (-1: bad token id or expert)  [T * top]
//   tile_expert[i]  = expert of tile i, -1 for unused tiles     [n_tiles], n_tiles >= ceil(T top / tile) + E
// Which row of its expert's range a pair gets depends on timing; no result depends on it, since every row
// of the grouped products is computed for itself.
// ---------------------------------------------------------------------------
__global__ void expert_plan_kernel(const int* __restrict__ ids, const int* __restrict__ table, int T, int V, int top,
                                   int E, int tile, int n_tiles, int* __restrict__ row_token, int* __restrict__ pair_row,
                                   int* __restrict__ tile_expert, unsigned* err) {
    extern __shared__ int sh[];
    int* count = sh;            // [E]
    int* start = sh + E;        // [E]
    int* cursor = sh + 2 * E;   // [E]
    const int tid = threadIdx.x, P = T * top;
    for (int e = tid; e < E; e += blockDim.x) count[e] = cursor[e] = 0;
    for (int i = tid; i < n_tiles * tile; i += blockDim.x) row_token[i] = -1;
    for (int i = tid; i < n_tiles; i += blockDim.x) tile_expert[i] = -1;
    __syncthreads();
    for (int p = tid; p < P; p += blockDim.x) {
        const int id = ids[p / top];
        int e = -1;
        if (id >= 0 && id < V) e = table[(size_t)id * top + p % top];
        if (e < 0 || e >= E) {
            atomicOr(err, AIE_DEV_TOKEN_OOB);
            continue;
        }
        atomicAdd(&count[e], 1);
    }
    __syncthreads();
    if (tid == 0) {
        int at = 0;
        for (int e = 0; e < E; ++e) {
            start[e] = at * tile;
            const int nt = (count[e] + tile - 1) / tile;
            for (int i = 0; i < nt && at + i < n_tiles; ++i) tile_expert[at + i] = e;
            at += nt;
        }
    }
    __syncthreads();
    for (int p = tid; p < P; p += blockDim.x) {
        const int id = ids[p / top];
        int e = -1;
        if (id >= 0 && id < V) e = table[(size_t)id * top + p % top];
        if (e < 0 || e >= E) {
            pair_row[p] = -1;
            continue;
        }
        const int row = start[e] + atomicAdd(&cursor[e], 1);
        pair_row[p] = row;
        if (row < n_tiles * tile) row_token[row] = p / top;
    }
}

extern "C" int aie_expert_plan(const int* ids, const int* table, int T, int V, int top, int E, int tile, int n_tiles,
                               int* row_token, int* pair_row, int* tile_expert, unsigned* err, cudaStream_t st) {
    if (T <= 0) return 0;
    if (top <= 0 || E <= 0 || tile <= 0 || (long long)n_tiles * tile < (long long)T * top) return AIE_BAD_ARG;
    if ((size_t)3 * E * sizeof(int) > 40000) return AIE_UNSUPPORTED;
    expert_plan_kernel<<<1, 1024, 3 * E * sizeof(int), st>>>(ids, table, T, V, top, E, tile, n_tiles, row_token, pair_row,
                                                              tile_expert, err);
    AIE_LAUNCH_CHECK();
}

// out[t] = w * sum_s y[pair_row[t top + s]]  (+ shared[t] * sigmoid(gate[t]))        float32
__global__ void expert_combine_kernel(const float* __restrict__ y, const int* __restrict__ pair_row, int top, float w,
                                      const float* __restrict__ shared, const float* __restrict__ gate, int ld_gate,
                                      float* __restrict__ out, int D) {
    const int t = blockIdx.x;
    float sg = 0.f;
    if (shared) sg = 1.0f / (1.0f + expf(-gate[(size_t)t * ld_gate]));
    for (int c = threadIdx.x; c < D; c += blockDim.x) {
        float acc = 0.f;
        for (int s = 0; s < top; ++s) {
            const int row = pair_row[(size_t)t * top + s];
            if (row >= 0) acc = fmaf(w, y[(size_t)row * D + c], acc);
        }
        if (shared) acc = fmaf(shared[(size_t)t * D + c], sg, acc);
        out[(size_t)t * D + c] = acc;
    }
}

extern "C" int aie_expert_combine(const float* y, const int* pair_row, int top, float w, const float* shared,
                                  const float* gate, int ld_gate, float* out, int T, int D, cudaStream_t st) {
    if (T <= 0) return 0;
    if (D <= 0 || top <= 0) return AIE_BAD_ARG;
    expert_combine_kernel<<<T, 256, 0, st>>>(y, pair_row, top, w, shared, gate, ld_gate, out, D);
    AIE_LAUNCH_CHECK();
}

// out[r] = src[rows[r]] (zeros where rows[r] < 0): the step's rows in the order of a grouping
template <typename T>
__global__ void gather_rows_kernel(const T* __restrict__ src, const int* __restrict__ rows, T* __restrict__ out, int D) {
    const int r = blockIdx.x, s = rows[r];
    for (int c = threadIdx.x; c < D; c += blockDim.x)
        out[(size_t)r * D + c] = s >= 0 ? src[(size_t)s * D + c] : from_f32<T>(0.f);
}

extern "C" int aie_gather_rows(const void* src, const int* rows, void* out, int dtype, int n, int D, cudaStream_t st) {
    if (n <= 0) return 0;
    if (D <= 0) return AIE_BAD_ARG;
    if (dtype == AIE_F32)
        gather_rows_kernel<float><<<n, 256, 0, st>>>((const float*)src, rows, (float*)out, D);
    else if (dtype == AIE_BF16)
        gather_rows_kernel<bf16><<<n, 256, 0, st>>>((const bf16*)src, rows, (bf16*)out, D);
    else
        return AIE_BAD_ARG;
    AIE_LAUNCH_CHECK();
}
