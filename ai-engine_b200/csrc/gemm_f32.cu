// True float32 matrix product on the CUDA cores (FMA; no tensor cores, no TF32):
//   C[M, N] = A[M, K] . W[N, K]^T        (weights as stored by HF: [out, in])
// It is the 32-bit path of every projection and of the LM head.  Each output
// element is one thread's running sum over k = 0 .. K-1 in that order, so a
// row's result does not depend on M: the same token gives the same bits
// whatever else is in the batch.
// The reference multiplies x[B,S,in] by a weight kept as [in,out]
// (crates/ai-engine-runtime/src/arch/linear.rs:106-123); the product is the same.
#include "common.cuh"

#define BM 64
#define BN 64
#define BK 16

template <typename AT, typename WT, typename OT>
__global__ void __launch_bounds__(256)
gemm_f32_kernel(const AT* __restrict__ A, const WT* __restrict__ W, OT* __restrict__ C,
                const int* __restrict__ a_rows, const int* __restrict__ tile_w, int M, int N, int K, int lda,
                int ldc, long long a_bs, long long w_bs, long long c_bs) {
    __shared__ float As[BK][BM + 4];
    __shared__ float Ws[BK][BN + 4];
    const int tid = threadIdx.x;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    // a batch of products (blockIdx.z), or one weight per tile of rows (tile_w: -1 = the tile is empty)
    A += (long long)blockIdx.z * a_bs;
    C += (long long)blockIdx.z * c_bs;
    if (tile_w) {
        const int e = tile_w[blockIdx.y];
        if (e < 0) return;
        W += (long long)e * w_bs;
    } else {
        W += (long long)blockIdx.z * w_bs;
    }
    const int tm = (tid / 16) * 4, tn = (tid % 16) * 4;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

    // loader mapping: 64 rows x 16 k per tile, 256 threads -> 4 consecutive k each
    const int lr = tid / 4, lk = (tid % 4) * 4;
    const int am = m0 + lr, wn = n0 + lr;
    const AT* arow = nullptr;
    if (am < M) {
        const int r = a_rows ? a_rows[am] : am;
        if (r >= 0) arow = A + (size_t)r * lda;
    }
    const WT* wrow = wn < N ? W + (size_t)wn * K : nullptr;

    for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int k = k0 + lk + j;
            As[lk + j][lr] = (arow && k < K) ? to_f32<AT>(arow[k]) : 0.f;
            Ws[lk + j][lr] = (wrow && k < K) ? to_f32<WT>(wrow[k]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < BK; ++k) {
            float a[4], w[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = As[k][tm + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) w[j] = Ws[k][tn + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int m = m0 + tm + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tn + j;
            if (n < N) C[(size_t)m * ldc + n] = from_f32<OT>(acc[i][j]);
        }
    }
}

template <typename AT, typename WT>
static int gemm_f32_go(const void* A, const void* W, void* C, int c_dtype, const int* a_rows, const int* tile_w,
                       int M, int N, int K, int lda, int ldc, int batch, long long a_bs, long long w_bs,
                       long long c_bs, cudaStream_t stream) {
    dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM, batch);
    if (grid.y > 65535 || batch > 65535) return AIE_UNSUPPORTED;
    if (c_dtype == AIE_F32)
        gemm_f32_kernel<AT, WT, float><<<grid, 256, 0, stream>>>((const AT*)A, (const WT*)W, (float*)C, a_rows, tile_w,
                                                                 M, N, K, lda, ldc, a_bs, w_bs, c_bs);
    else if (c_dtype == AIE_BF16)
        gemm_f32_kernel<AT, WT, bf16><<<grid, 256, 0, stream>>>((const AT*)A, (const WT*)W, (bf16*)C, a_rows, tile_w,
                                                                M, N, K, lda, ldc, a_bs, w_bs, c_bs);
    else
        return AIE_BAD_ARG;
    AIE_LAUNCH_CHECK();
}

// The general form.  A [M, lda] (float32 or bfloat16, widened on load), W [N, K], C [M, ldc] (float32 or
// bfloat16, rounded once at the store).  a_rows (optional): row m of the product reads A[a_rows[m]] (a
// negative entry reads zeros).  batch > 1: `batch` independent products whose operands lie a_bs / w_bs / c_bs
// elements apart (per-head projections).  tile_w (optional, batch == 1): rows 64 i .. 64 i + 63 of the product
// use the weight W + tile_w[i] * w_bs (rows grouped by expert; -1 skips the tile).
extern "C" int aie_gemm_f32_ex(const void* A, int a_dtype, const void* W, int w_dtype, void* C, int c_dtype,
                               const int* a_rows, const int* tile_w, int M, int N, int K, int lda, int ldc,
                               int batch, long long a_bs, long long w_bs, long long c_bs, cudaStream_t stream) {
    if (M <= 0 || N <= 0 || batch <= 0) return 0;
    if (K <= 0 || (tile_w && batch != 1)) return AIE_BAD_ARG;
#define GO(AT, WT) return gemm_f32_go<AT, WT>(A, W, C, c_dtype, a_rows, tile_w, M, N, K, lda, ldc, batch, a_bs, w_bs, c_bs, stream)
    if (a_dtype == AIE_F32 && w_dtype == AIE_F32) GO(float, float);
    if (a_dtype == AIE_F32 && w_dtype == AIE_BF16) GO(float, bf16);
    if (a_dtype == AIE_BF16 && w_dtype == AIE_F32) GO(bf16, float);
    if (a_dtype == AIE_BF16 && w_dtype == AIE_BF16) GO(bf16, bf16);
#undef GO
    return AIE_BAD_ARG;
}

// a_rows (optional): row m of the product reads A[a_rows[m]] (the LM head runs
// only on the rows whose logits are wanted).
extern "C" int aie_gemm_f32(const float* A, const void* W, int w_dtype, float* C, const int* a_rows,
                            int M, int N, int K, int ldc, cudaStream_t stream) {
    return aie_gemm_f32_ex(A, AIE_F32, W, w_dtype, C, AIE_F32, a_rows, nullptr, M, N, K, K, ldc, 1, 0, 0, 0, stream);
}
