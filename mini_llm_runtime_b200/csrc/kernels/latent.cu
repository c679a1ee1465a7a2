// Attention whose keys and values are projections of ONE small vector per token (the latent), so that
// only that vector is cached:  k_h = Uk_h c,  v_h = Uv_h c.
//
// The scores  q_h . (Uk_h c)  equal  (Uk_h^T q_h) . c,  and  sum_j p_j Uv_h c_j = Uv_h (sum_j p_j c_j):  with the
// query taken through Uk_h^T first and the result through Uv_h afterwards, attention runs on the cached latents
// themselves, as keys and as values of one shared kv head (`attention_masked.cu` with shared_kv).  Here are the
// two row-wise pieces around it:
//
//   mlr_latent_cache    c = rmsnorm(row of the down projection) * weight, float32 math, into the token's place
//                       of its page ([page][token_in_page][rank], one kv head, keys only)
//   mlr_head_project    y[m, h, :] = x[m, h, :] W_h,  W [heads, A, B] row-major, float32 sums in the order a = 0..A-1 (the
//                       float32 path and odd sizes; bfloat16 rows on 16-byte borders take `mlr_batched_product_bf16` of experts.cu)
#include "common.cuh"

namespace {

constexpr int kThreads = 128;
constexpr int kRows = 8;

template <typename T>
__global__ void __launch_bounds__(kThreads) latent_cache_kernel(const T* in, long long ld, const T* weight_t, const float* weight_f, float eps,
                                                                int rank, T* cache, int num_pages, const int* positions,
                                                                const int* segment_of_row, const int* block_table, int table_stride,
                                                                int page_size, int* status) {
    mlr_grid_wait();
    __shared__ float scratch[32];
    const int row = blockIdx.x;
    const int position = positions[row];
    const int page = block_table[static_cast<size_t>(segment_of_row[row]) * table_stride + position / page_size];
    if (page < 0 || page >= num_pages) {
        if (threadIdx.x == 0 && status) atomicOr(status, MLR_STATUS_BAD_PAGE);
        return;
    }
    const T* x = in + static_cast<size_t>(row) * ld;
    float sum = 0.0f;
    for (int c = threadIdx.x; c < rank; c += kThreads) {
        const float v = mlr_load(x, c);
        sum = fmaf(v, v, sum);
    }
    const float inv = 1.0f / sqrtf(mlr_block_sum(sum, scratch) / static_cast<float>(rank) + eps);
    T* dst = cache + (static_cast<size_t>(page) * page_size + position % page_size) * rank;
    for (int c = threadIdx.x; c < rank; c += kThreads) {
        const float w = weight_f ? weight_f[c] : mlr_load(weight_t, c);
        mlr_store(dst, c, mlr_load(x, c) * inv * w);
    }
    mlr_grid_dependents_may_start();
}

// A block: kRows rows x one head x 128 outputs; the rows' inputs of that head as float32 in shared memory.
template <typename T>
__global__ void __launch_bounds__(kThreads) head_project_kernel(const T* x, long long ldx, const T* w, T* y, long long ldy, int rows, int A, int B) {
    mlr_grid_wait();
    extern __shared__ __align__(16) float xs[];          // [kRows][A]
    const int row0 = blockIdx.x * kRows, head = blockIdx.y, b = blockIdx.z * kThreads + threadIdx.x;
    const int n = min(kRows, rows - row0);
    for (int i = threadIdx.x; i < kRows * A; i += kThreads) {
        const int r = i / A, a = i % A;
        xs[i] = r < n ? mlr_load(x + static_cast<size_t>(row0 + r) * ldx + static_cast<size_t>(head) * A, a) : 0.0f;
    }
    __syncthreads();
    mlr_grid_dependents_may_start();
    if (b >= B) return;
    const T* wh = w + static_cast<size_t>(head) * A * B + b;
    float acc[kRows] = {};
    int a = 0;
    for (; a + 8 <= A; a += 8) {          // eight loads of the matrix in flight
        float v[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = mlr_load(wh, static_cast<size_t>(a + i) * B);
#pragma unroll
        for (int i = 0; i < 8; ++i)
#pragma unroll
            for (int r = 0; r < kRows; ++r) acc[r] = fmaf(xs[r * A + a + i], v[i], acc[r]);
    }
    for (; a < A; ++a) {
        const float v = mlr_load(wh, static_cast<size_t>(a) * B);
#pragma unroll
        for (int r = 0; r < kRows; ++r) acc[r] = fmaf(xs[r * A + a], v, acc[r]);
    }
#pragma unroll
    for (int r = 0; r < kRows; ++r)
        if (r < n) mlr_store(y + static_cast<size_t>(row0 + r) * ldy + static_cast<size_t>(head) * B, b, acc[r]);
}

}  // namespace

// in: the rows of the down projection (row stride ld, `rank` values each); weight: [rank] in float32 (weight_f32) or the
// activations' precision; cache: [pages, page_size * rank] of the activations' precision.
MLR_API int mlr_latent_cache(const void* in, long long ld, int act_bf16, const void* weight, int weight_f32, float eps, int rank, void* cache,
                             int num_pages, const int* positions, const int* segment_of_row, const int* block_table, int table_stride,
                             int page_size, int rows, int* status, cudaStream_t stream) {
    MLR_REQUIRE(in && weight && cache && positions && segment_of_row && block_table && rank > 0 && page_size > 0 && num_pages > 0,
                "latent_cache: bad arguments");
    if (rows <= 0) return 0;
    const float* wf = weight_f32 ? static_cast<const float*>(weight) : nullptr;
    if (act_bf16)
        mlr_launch((latent_cache_kernel<__nv_bfloat16>), dim3(rows), dim3(kThreads), 0, stream, static_cast<const __nv_bfloat16*>(in), ld,
                   static_cast<const __nv_bfloat16*>(weight), wf, eps, rank, static_cast<__nv_bfloat16*>(cache), num_pages, positions,
                   segment_of_row, block_table, table_stride, page_size, status);
    else
        mlr_launch((latent_cache_kernel<float>), dim3(rows), dim3(kThreads), 0, stream, static_cast<const float*>(in), ld,
                   static_cast<const float*>(weight), wf, eps, rank, static_cast<float*>(cache), num_pages, positions, segment_of_row,
                   block_table, table_stride, page_size, status);
    return mlr_launched("latent_cache");
}

// x: [rows, heads * A] (row stride ldx), w: [heads, A, B], y: [rows, heads * B] (row stride ldy), all in the activations' precision.
MLR_API int mlr_head_project(const void* x, long long ldx, const void* w, void* y, long long ldy, int act_bf16, int rows, int heads, int A, int B,
                             cudaStream_t stream) {
    MLR_REQUIRE(x && w && y && heads > 0 && heads <= 65535 && A > 0 && B > 0, "head_project: bad arguments");
    const size_t shared = sizeof(float) * kRows * static_cast<size_t>(A);
    MLR_REQUIRE(shared <= 200 * 1024, "head_project: %d inputs per head do not fit shared memory", A);
    if (rows <= 0) return 0;
    const dim3 grid((rows + kRows - 1) / kRows, heads, (B + kThreads - 1) / kThreads);
    if (act_bf16) {
        if (shared > 48 * 1024) cudaFuncSetAttribute(head_project_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(shared));
        mlr_launch((head_project_kernel<__nv_bfloat16>), dim3(grid), dim3(kThreads), shared, stream, static_cast<const __nv_bfloat16*>(x), ldx,
                   static_cast<const __nv_bfloat16*>(w), static_cast<__nv_bfloat16*>(y), ldy, rows, A, B);
    } else {
        if (shared > 48 * 1024) cudaFuncSetAttribute(head_project_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(shared));
        mlr_launch((head_project_kernel<float>), dim3(grid), dim3(kThreads), shared, stream, static_cast<const float*>(x), ldx,
                   static_cast<const float*>(w), static_cast<float*>(y), ldy, rows, A, B);
    }
    return mlr_launched("head_project");
}
