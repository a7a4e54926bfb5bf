// Tensor-core attention over the compressed cache (bfloat16 rows [latent (rank) | rotated key part (rot)], one per
// token, shared by all heads): see latent_attention.cu for the formula.  All heads of a token multiply the same
// cache rows, so the heads are the rows of the products: one CTA owns one query token and a group of 16 heads
// (one m16 tile of mma.sync m16n8k16, bf16 in, float32 accumulate) and walks the token's visible keys in chunks
// of 64 that start at multiples of 64 of the absolute key position (a row's additions depend on its position
// only, not on how the prompt was cut or on the batch).  A CTA of a prompt's portion takes TQ = 4 consecutive tokens
// of one request (four warps each): they share the gathered cache rows, whose traffic from L2 bounds the kernel,
// and differ only in their masks.
//
// Per chunk: the 64 cache rows are gathered page by page into shared memory by 16-byte cp.async copies (rows
// outside the mask or the block table are zero-filled, so a probability of 0 never meets an unwritten row);
// S = Q K^T with the chunk's keys split over the four warps; scores, mask, running maximum and sum in float32
// in shared memory (eight threads a row); O += P V with the latent's columns split over the four warps, V being
// the first `rank` columns of the same rows (ldmatrix.trans).  Few tokens in a step (decoding) cut each token's
// chunks into `splits` parts that run as CTAs of their own and leave (maximum, sum, unnormalised output) for a
// joining kernel.
#include "attention_prefill.cuh"

#define LT_KEYS 64
#define LT_ROWS 16
#define LT_THREADS 128

template <int CW, int TQ>      // latent columns per warp (rank = 4 CW); tokens per CTA
__global__ void __launch_bounds__(LT_THREADS * TQ)
latent_attention_tc_kernel(const float* __restrict__ q_full, const bf16* __restrict__ pages, bf16* __restrict__ out,
                           float* __restrict__ part_o, float* __restrict__ part_ml, const int* __restrict__ tiles,
                           const int* __restrict__ q_start, const int* __restrict__ q_len,
                           const int* __restrict__ ctx_len, const int* __restrict__ block_table, int bt_width,
                           int num_pages, int P, int H, int dk, int window, float scale, int splits, unsigned* err) {
    constexpr int RANK = 4 * CW, NT = CW / 8, THREADS = LT_THREADS * TQ;
    extern __shared__ __align__(16) unsigned char lt_raw[];
    const int SK = dk + 8;                                        // padded row: ldmatrix rows fall on different banks
    bf16* q_all = reinterpret_cast<bf16*>(lt_raw);                // [TQ][16][SK]
    bf16* k_s = q_all + TQ * LT_ROWS * SK;                        // [64][SK]
    bf16* p_all = k_s + LT_KEYS * SK;                             // [TQ][16][64 + 8]
    float* s_all = reinterpret_cast<float*>(p_all + TQ * LT_ROWS * (LT_KEYS + 8));     // [TQ][16][64 + 1]
    float* m_all = s_all + TQ * LT_ROWS * (LT_KEYS + 1);          // [TQ][16] running maximum
    float* l_all = m_all + TQ * LT_ROWS;                          // [TQ][16] running sum
    float* c_all = l_all + TQ * LT_ROWS;                          // [TQ][16] correction of this chunk

    const int row = tiles[2 * blockIdx.x], off = tiles[2 * blockIdx.x + 1];
    const int h0 = blockIdx.y * LT_ROWS, part = blockIdx.z;
    const int tid = threadIdx.x, tq = tid / LT_THREADS, ltid = tid % LT_THREADS, warp = (tid >> 5) & 3, lane = tid & 31;
    const int n_act = min(TQ, q_len[row] - off);                  // tokens of this CTA that exist
    const int pos_first = ctx_len[row] + off, pos_last = pos_first + n_act - 1;
    const int t = q_start[row] + off + tq;
    const bool active = tq < n_act;
    const int pos = active ? pos_first + tq : -1;                 // a token that does not exist sees no key
    int lo = 0, lo_first = 0;
    if (window > 0 && pos - window + 1 > 0) lo = pos - window + 1;
    if (window > 0 && pos_first - window + 1 > 0) lo_first = pos_first - window + 1;
    const int first_chunk = lo_first / LT_KEYS, n_chunks = pos_last / LT_KEYS - first_chunk + 1;
    const int per = (n_chunks + splits - 1) / splits;
    const int c_begin = first_chunk + part * per, c_end = min(first_chunk + n_chunks, c_begin + per);
    bf16* q_s = q_all + tq * LT_ROWS * SK;
    bf16* p_s = p_all + tq * LT_ROWS * (LT_KEYS + 8);
    float* s_s = s_all + tq * LT_ROWS * (LT_KEYS + 1);
    float* m_s = m_all + tq * LT_ROWS;
    float* l_s = l_all + tq * LT_ROWS;
    float* c_s = c_all + tq * LT_ROWS;

    // the 16 heads' queries, rounded to bfloat16 (rows past the last head are zero)
    for (int r = warp; r < LT_ROWS; r += 4) {                     // a warp converts whole rows, four elements a lane
        const bool on = active && h0 + r < H;
        const float* src = q_full + ((size_t)t * H + h0 + r) * dk;
        for (int c = lane * 4; c < dk; c += 128) {
            const float4 v = on ? *reinterpret_cast<const float4*>(src + c) : make_float4(0.f, 0.f, 0.f, 0.f);
            *reinterpret_cast<uint2*>(q_s + r * SK + c) = make_uint2(pack_bf16(v.x, v.y), pack_bf16(v.z, v.w));
        }
    }
    if (ltid < LT_ROWS) {
        m_s[ltid] = -INFINITY;
        l_s[ltid] = 0.f;
    }
    float acc[NT][4];
#pragma unroll
    for (int i = 0; i < NT; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;
    const int pieces = dk / 8;                                    // 16-byte pieces a row

    for (int ch = c_begin; ch < c_end; ++ch) {
        const int k0 = ch * LT_KEYS;
        __syncthreads();                                          // the previous chunk's rows and probabilities are done with
        // a warp copies whole rows: one look-up of the page per row, the lanes take the row's 16-byte pieces
        for (int j = tid >> 5; j < LT_KEYS; j += THREADS / 32) {
            const int kp = k0 + j;
            bool ok = kp >= lo_first && kp <= pos_last;
            const bf16* src = pages;
            if (ok) {
                const int pidx = kp / P;
                const int page = pidx < bt_width ? block_table[(size_t)row * bt_width + pidx] : -1;
                if (page < 0 || page >= num_pages) {
                    if (lane == 0) atomicOr(err, AIE_DEV_PAGE_OOB);
                    ok = false;
                } else {
                    src = pages + ((size_t)page * P + (kp - pidx * P)) * dk;
                }
            }
            for (int c = lane; c < pieces; c += 32) cp_async16(k_s + j * SK + c * 8, ok ? src + c * 8 : pages, ok);
        }
        cp_async_commit();
        cp_async_wait<0>();
        __syncthreads();

        // S = Q K^T: warp w multiplies keys 16 w .. 16 w + 15
        // two sets of accumulators take alternate k steps, so that a product does not wait for the one before it
        // and the fragments of the next step are on their way while this step multiplies
        float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
        float s2[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
        const bf16* qa = q_s + (lane & 15) * SK + (lane >> 4) * 8;
        // rows = keys; matrices: (keys 0-7, k 0-7), (keys 0-7, k 8-15), (keys 8-15, k 0-7), (keys 8-15, k 8-15)
        const bf16* kb = k_s + (warp * 16 + (lane & 7) + ((lane >> 4) << 3)) * SK + ((lane >> 3) & 1) * 8;
        int kk = 0;
#pragma unroll 2
        for (; kk + 32 <= dk; kk += 32) {
            unsigned a[4], c[4], b0, b1, b2, b3, d0, d1, d2, d3;
            ldsm_x4(a[0], a[1], a[2], a[3], qa + kk);
            ldsm_x4(b0, b1, b2, b3, kb + kk);
            ldsm_x4(c[0], c[1], c[2], c[3], qa + kk + 16);
            ldsm_x4(d0, d1, d2, d3, kb + kk + 16);
            mma16816(s[0], a, b0, b1);
            mma16816(s[1], a, b2, b3);
            mma16816(s2[0], c, d0, d1);
            mma16816(s2[1], c, d2, d3);
        }
        if (kk < dk) {
            unsigned a[4], b0, b1, b2, b3;
            ldsm_x4(a[0], a[1], a[2], a[3], qa + kk);
            ldsm_x4(b0, b1, b2, b3, kb + kk);
            mma16816(s[0], a, b0, b1);
            mma16816(s[1], a, b2, b3);
        }
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            s[0][e] += s2[0][e];
            s[1][e] += s2[1][e];
        }
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
            const int col = warp * 16 + nt * 8 + (lane & 3) * 2, r0 = lane >> 2;
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int r = r0 + (e >> 1) * 8, c = col + (e & 1), kp = k0 + c;
                s_s[r * (LT_KEYS + 1) + c] = (kp >= lo && kp <= pos) ? s[nt][e] * scale : -INFINITY;
            }
        }
        __syncthreads();
        // running softmax: eight threads a row, eight keys a thread
        {
            const int r = ltid >> 3, g = ltid & 7;
            float v[8], mx = -INFINITY;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                v[i] = s_s[r * (LT_KEYS + 1) + g * 8 + i];
                mx = fmaxf(mx, v[i]);
            }
#pragma unroll
            for (int o = 4; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
            const float m_old = m_s[r], m_new = fmaxf(m_old, mx);
            float sum = 0.f;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const float p = (m_new == -INFINITY || v[i] == -INFINITY) ? 0.f : expf(v[i] - m_new);
                const bf16 pb = __float2bfloat16_rn(p);
                p_s[r * (LT_KEYS + 8) + g * 8 + i] = pb;
                sum += __bfloat162float(pb);          // the sum of what the product will multiply
            }
#pragma unroll
            for (int o = 4; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
            __syncwarp();
            if (g == 0) {
                const float corr = (m_old == -INFINITY) ? 0.f : expf(m_old - m_new);
                c_s[r] = corr;
                l_s[r] = l_s[r] * corr + sum;
                m_s[r] = m_new;
            }
        }
        __syncthreads();
        // O = O * corr + P V: warp w owns latent columns CW w .. CW w + CW - 1
        {
            const float ca = c_s[lane >> 2], cb = c_s[(lane >> 2) + 8];
#pragma unroll
            for (int i = 0; i < NT; ++i) {
                acc[i][0] *= ca;
                acc[i][1] *= ca;
                acc[i][2] *= cb;
                acc[i][3] *= cb;
            }
#pragma unroll
            for (int kk = 0; kk < LT_KEYS; kk += 16) {
                unsigned a[4];
                ldsm_x4(a[0], a[1], a[2], a[3], p_s + (lane & 15) * (LT_KEYS + 8) + kk + (lane >> 4) * 8);
#pragma unroll
                for (int np = 0; np < NT / 2; ++np) {
                    unsigned b0, b1, b2, b3;
                    // rows = keys kk .. kk + 15 of V; matrices: (k 0-7, n 0-7), (k 8-15, n 0-7), (k 0-7, n 8-15), (k 8-15, n 8-15)
                    ldsm_x4_t(b0, b1, b2, b3, k_s + (kk + (lane & 7) + ((lane >> 3) & 1) * 8) * SK + warp * CW + np * 16 + (lane >> 4) * 8);
                    mma16816(acc[2 * np], a, b0, b1);
                    mma16816(acc[2 * np + 1], a, b2, b3);
                }
            }
        }
    }
    __syncthreads();
    const int ra = lane >> 2, rb = ra + 8;
    if (!active) return;
    if (splits == 1) {
        const float ia = l_s[ra] > 0.f ? 1.0f / l_s[ra] : 0.f, ib = l_s[rb] > 0.f ? 1.0f / l_s[rb] : 0.f;
#pragma unroll
        for (int i = 0; i < NT; ++i) {
            const int col = warp * CW + i * 8 + (lane & 3) * 2;
            if (h0 + ra < H)
                *reinterpret_cast<unsigned*>(out + ((size_t)t * H + h0 + ra) * RANK + col) = pack_bf16(acc[i][0] * ia, acc[i][1] * ia);
            if (h0 + rb < H)
                *reinterpret_cast<unsigned*>(out + ((size_t)t * H + h0 + rb) * RANK + col) = pack_bf16(acc[i][2] * ib, acc[i][3] * ib);
        }
    } else {
        // a part leaves its unnormalised output, maximum and sum (an empty part: sum 0)
#pragma unroll
        for (int i = 0; i < NT; ++i) {
            const int col = warp * CW + i * 8 + (lane & 3) * 2;
            if (h0 + ra < H)
                *reinterpret_cast<float2*>(part_o + (((size_t)t * H + h0 + ra) * splits + part) * RANK + col) = make_float2(acc[i][0], acc[i][1]);
            if (h0 + rb < H)
                *reinterpret_cast<float2*>(part_o + (((size_t)t * H + h0 + rb) * splits + part) * RANK + col) = make_float2(acc[i][2], acc[i][3]);
        }
        if (ltid < LT_ROWS && h0 + ltid < H) {
            float* ml = part_ml + (((size_t)t * H + h0 + ltid) * splits + part) * 2;
            ml[0] = m_s[ltid];
            ml[1] = l_s[ltid];
        }
    }
}

// out[t, h] = sum_p w_p O_p / sum_p w_p l_p with w_p = exp(m_p - max m), parts in order
__global__ void latent_join_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                   bf16* __restrict__ out, int splits, int rank) {
    const size_t th = blockIdx.x;
    const float* ml = part_ml + th * splits * 2;
    float mx = -INFINITY;
    for (int p = 0; p < splits; ++p)
        if (ml[2 * p + 1] > 0.f) mx = fmaxf(mx, ml[2 * p]);
    float den = 0.f;
    for (int p = 0; p < splits; ++p)
        if (ml[2 * p + 1] > 0.f) den += expf(ml[2 * p] - mx) * ml[2 * p + 1];
    const float inv = den > 0.f ? 1.0f / den : 0.f;
    for (int c = threadIdx.x; c < rank; c += blockDim.x) {
        float acc = 0.f;
        for (int p = 0; p < splits; ++p)
            if (ml[2 * p + 1] > 0.f) acc = fmaf(expf(ml[2 * p] - mx), part_o[(th * splits + p) * rank + c], acc);
        out[th * rank + c] = __float2bfloat16_rn(acc * inv);
    }
}

// q_full [T, H, dk] float32; pages [num_pages, P, dk] bfloat16; out [T, H, rank] bfloat16.  tiles [n_tiles, 2] =
// (request row, offset among the tokens it brings) of units of `tq` tokens (1 or 4).  Takes rank = 64 .. 512 in
// steps of 64 and dk a multiple of 16 (else AIE_UNSUPPORTED: the caller takes the plain kernel).  splits > 1 needs
// part_o [T, H, splits, rank] and part_ml [T, H, splits, 2] float32.
extern "C" int aie_latent_attention_tc(const float* q_full, const void* pages, void* out, float* part_o, float* part_ml,
                                       const int* tiles, int n_tiles, int tq, const int* q_start, const int* q_len,
                                       const int* ctx_len, const int* block_table, int bt_width,
                                       int num_pages, int P, int T, int H, int rank, int dk, int window, float scale,
                                       int splits, unsigned* err, cudaStream_t st) {
    if (T <= 0 || n_tiles <= 0) return 0;
    if (rank < 64 || rank > 512 || rank % 64 || dk % 16 || dk < rank || dk > 1024 || H <= 0) return AIE_UNSUPPORTED;
    if (splits < 1 || splits > 64 || (splits > 1 && (!part_o || !part_ml)) || (tq != 1 && tq != 4)) return AIE_BAD_ARG;
    const int SK = dk + 8;
    const size_t smem = (size_t)(tq * LT_ROWS + LT_KEYS) * SK * 2 + (size_t)tq * LT_ROWS * (LT_KEYS + 8) * 2 +
                        (size_t)tq * (LT_ROWS * (LT_KEYS + 1) + 3 * LT_ROWS) * 4;
    if (smem > 220 * 1024) return AIE_UNSUPPORTED;
    dim3 grid(n_tiles, (H + LT_ROWS - 1) / LT_ROWS, splits);
    if (grid.y > 65535) return AIE_UNSUPPORTED;
#define GO1(CWV, TQV)                                                                                                 \
    {                                                                                                                 \
        auto kern = latent_attention_tc_kernel<CWV, TQV>;                                                             \
        cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);                           \
        kern<<<grid, LT_THREADS * TQV, smem, st>>>(q_full, (const bf16*)pages, (bf16*)out, part_o, part_ml, tiles,    \
                                                   q_start, q_len, ctx_len, block_table, bt_width, num_pages, P, H,   \
                                                   dk, window, scale, splits, err);                                   \
    }
#define GO(CWV)                                                                                                       \
    case CWV:                                                                                                         \
        if (tq == 1) GO1(CWV, 1) else GO1(CWV, 4)                                                                     \
        break;
    switch (rank / 4) {
        GO(16) GO(32) GO(48) GO(64) GO(80) GO(96) GO(112) GO(128)
        default: return AIE_UNSUPPORTED;
    }
#undef GO
#undef GO1
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return (int)e;
    if (splits > 1) latent_join_kernel<<<T * H, 128, 0, st>>>(part_o, part_ml, (bf16*)out, splits, rank);
    AIE_LAUNCH_CHECK();
}
