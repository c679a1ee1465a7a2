// A residual stream kept as several copies (hyper-connections), and the embedding that starts it.
//
//   The stream of a token is S vectors x_1 .. x_S of `width` values (float32, [rows, S * width]).  A
//   sub-layer reads  u = sum_s a[s] x_s,  works on norm(u), and its result y goes back as
//       x_t <- sum_s B[s, t] x_s + c[t] * (g .* y)        (all t from the old copies; g a vector, or none)
//   `mlr_streams_step` does the write of one sub-layer and the read (with the RMS norm) of the next in
//   one pass over the row: either half may be absent.  With S = 1, B = [[1]], c = [1], a = [1] it is the
//   ordinary residual add (scaled element by element) with the norm behind it.  Without `a` the read is
//   the plain sum of the copies (what a model's last norm takes).  Everything is float32; only the
//   normed activations leave in the activation precision.
//
//   `mlr_embed_hashed`: x = table[id] * scale + pairs[(prev * m_prev + id * m_cur) mod buckets], the same
//   vector into every copy of the stream; a sequence's first token takes row `buckets` of `pairs`.
//   The token before a row is the row above it, or, for the first row of a step's segment, what the
//   request's state slot holds; the slot then takes the segment's last token.
#include "common.cuh"

namespace {

constexpr int kMaxStreams = 16;
constexpr int kThreads = 256;

struct StreamWeights {
    float mix[kMaxStreams * kMaxStreams];   // [from][to]
    float out[kMaxStreams];
    float in[kMaxStreams];
};

// S: the number of copies when it is at most 8 (weights in registers, loops unrolled), or 0 for any number up to kMaxStreams
// (weights in shared memory).  V: columns a thread takes at a time (4 when the width and all strides allow 16-byte accesses).
template <typename TO, int S, int V>
__global__ void __launch_bounds__(kThreads) streams_step_kernel(float* h, const float* y, long long ld_y, const float* y_scale, const float* mix,
                                                                 const float* w_out, const float* w_in, const float* norm_weight, float eps,
                                                                 TO* out, long long ld_out, const int* rows, int width, int streams_given) {
    mlr_grid_wait();
    extern __shared__ __align__(16) float u[];          // [width]
    __shared__ float scratch[32];
    __shared__ StreamWeights w;
    constexpr int kCopies = S ? S : kMaxStreams;
    const int streams = S ? S : streams_given;
    const int row = rows ? rows[blockIdx.x] : blockIdx.x;
    if (threadIdx.x < streams * streams && mix) w.mix[threadIdx.x] = mix[threadIdx.x];
    if (threadIdx.x < streams) {
        if (w_out) w.out[threadIdx.x] = w_out[threadIdx.x];
        w.in[threadIdx.x] = w_in ? w_in[threadIdx.x] : 1.0f;
    }
    __syncthreads();
    // With a fixed S the weights move to registers (constant indices after unrolling).
    float rmix[S ? S * S : 1], rout[S ? S : 1], rin[S ? S : 1];
    if (S) {
#pragma unroll
        for (int i = 0; i < S * S; ++i) rmix[i] = y ? w.mix[i] : 0.0f;
#pragma unroll
        for (int i = 0; i < S; ++i) {
            rout[i] = y ? w.out[i] : 0.0f;
            rin[i] = w.in[i];
        }
    }
    float* x = h + static_cast<size_t>(row) * streams * width;
    const float* yrow = y ? y + static_cast<size_t>(row) * ld_y : nullptr;
    float squares = 0.0f;
    for (int c = threadIdx.x * V; c < width; c += kThreads * V) {
        float old[kCopies][V];
#pragma unroll
        for (int s = 0; s < kCopies; ++s) {
            if (s < streams) {
                if (V == 4) {
                    const float4 v = *reinterpret_cast<const float4*>(x + static_cast<size_t>(s) * width + c);
                    old[s][0] = v.x, old[s][1] = v.y, old[s][2] = v.z, old[s][V - 1] = v.w;
                } else {
                    old[s][0] = x[static_cast<size_t>(s) * width + c];
                }
            }
        }
        float sum[V];
#pragma unroll
        for (int e = 0; e < V; ++e) sum[e] = 0.0f;
        if (yrow) {
            float add[V];
#pragma unroll
            for (int e = 0; e < V; ++e) {
                add[e] = __ldcg(yrow + c + e);
                if (y_scale) add[e] *= y_scale[c + e];
            }
#pragma unroll
            for (int t = 0; t < kCopies; ++t) {
                if (t < streams) {
                    float value[V];
#pragma unroll
                    for (int e = 0; e < V; ++e) value[e] = 0.0f;
#pragma unroll
                    for (int s = 0; s < kCopies; ++s)
                        if (s < streams) {
                            const float m = S ? rmix[S ? s * S + t : 0] : w.mix[s * streams + t];
#pragma unroll
                            for (int e = 0; e < V; ++e) value[e] = fmaf(m, old[s][e], value[e]);
                        }
                    const float o = S ? rout[S ? t : 0] : w.out[t], in = S ? rin[S ? t : 0] : w.in[t];
#pragma unroll
                    for (int e = 0; e < V; ++e) {
                        value[e] = fmaf(o, add[e], value[e]);
                        sum[e] = fmaf(in, value[e], sum[e]);
                    }
                    if (V == 4) *reinterpret_cast<float4*>(x + static_cast<size_t>(t) * width + c) = make_float4(value[0], value[1], value[2], value[V - 1]);
                    else x[static_cast<size_t>(t) * width + c] = value[0];
                }
            }
        } else {
#pragma unroll
            for (int s = 0; s < kCopies; ++s)
                if (s < streams) {
                    const float in = S ? rin[S ? s : 0] : w.in[s];
#pragma unroll
                    for (int e = 0; e < V; ++e) sum[e] = fmaf(in, old[s][e], sum[e]);
                }
        }
        if (out) {
#pragma unroll
            for (int e = 0; e < V; ++e) {
                u[c + e] = sum[e];
                squares = fmaf(sum[e], sum[e], squares);
            }
        }
    }
    if (!out) {
        mlr_grid_dependents_may_start();
        return;
    }
    const float inv = 1.0f / sqrtf(mlr_block_sum(squares, scratch) / static_cast<float>(width) + eps);
    TO* orow = out + static_cast<size_t>(blockIdx.x) * ld_out;
    for (int c = threadIdx.x; c < width; c += kThreads) mlr_store(orow, c, u[c] * inv * (norm_weight ? norm_weight[c] : 1.0f));
    mlr_grid_dependents_may_start();
}

template <typename T>
__global__ void __launch_bounds__(kThreads) embed_hashed_kernel(float* h, const T* table, const T* pairs, const int* ids, const int* segment_of_row,
                                                                 const int* segment_info, int* state, long long state_stride, int width,
                                                                 int vocab, int streams, float scale, int buckets, int mul_prev, int mul_cur,
                                                                 int* status) {
    mlr_grid_wait();
    __shared__ int pair_row;
    const int row = blockIdx.x;
    const int id = ids[row];
    float* x = h + static_cast<size_t>(row) * streams * width;
    if (id < 0 || id >= vocab) {
        if (threadIdx.x == 0 && status) atomicOr(status, MLR_STATUS_BAD_INDEX);
        for (int c = threadIdx.x; c < streams * width; c += kThreads) x[c] = 0.0f;
        return;
    }
    if (threadIdx.x == 0) {
        pair_row = -1;
        if (pairs) {
            const int* info = segment_info + 4 * segment_of_row[row];
            const int first = info[0], count = info[1], start = info[2], slot = info[3];
            int* kept = state + static_cast<size_t>(slot) * state_stride;
            int prev;
            if (row == first) {
                prev = start == 0 ? -1 : *kept;
                // Only this block reads the slot in this step, so it is also the one that moves it on.
                *kept = ids[first + count - 1];
            } else {
                prev = ids[row - 1];
            }
            if (prev < 0) pair_row = buckets;
            else pair_row = static_cast<int>((static_cast<long long>(prev) * mul_prev + static_cast<long long>(id) * mul_cur) % buckets);
        }
    }
    __syncthreads();
    const T* trow = table + static_cast<size_t>(id) * width;
    const T* prow = pair_row >= 0 ? pairs + static_cast<size_t>(pair_row) * width : nullptr;
    for (int c = threadIdx.x; c < width; c += kThreads) {
        float value = mlr_load(trow, c) * scale;
        if (prow) value += mlr_load(prow, c);
        for (int s = 0; s < streams; ++s) x[static_cast<size_t>(s) * width + c] = value;
    }
    mlr_grid_dependents_may_start();
}

}  // namespace

// h: float32 [rows of the step, streams * width].  y (float32, row stride ld_y) with mix [streams, streams], w_out [streams] and
// optionally y_scale [width]: the write.  out (bfloat16 or float32 [count, width]) with norm_weight [width] (or null) and w_in
// [streams] (or null: the plain sum): the read.  rows: which rows of h the `count` blocks work on (null: 0 .. count-1); with
// `rows` the write must be absent (it would leave the other rows behind).
MLR_API int mlr_streams_step(float* h, const float* y, long long ld_y, const float* y_scale, const float* mix, const float* w_out,
                             const float* w_in, const float* norm_weight, float eps, void* out, long long ld_out, int out_bf16,
                             const int* rows, int count, int width, int streams, cudaStream_t stream) {
    MLR_REQUIRE(h && width > 0 && streams >= 1 && streams <= kMaxStreams, "streams_step: 1 to %d copies of the stream, got %d", kMaxStreams, streams);
    MLR_REQUIRE(y || out, "streams_step: neither a write nor a read");
    MLR_REQUIRE(!y || (mix && w_out && !rows), "streams_step: a write needs its weights and all rows");
    MLR_REQUIRE(static_cast<size_t>(width) * sizeof(float) <= 200 * 1024, "streams_step: a width of %d does not fit shared memory", width);
    if (count <= 0) return 0;
    const size_t shared = out ? static_cast<size_t>(width) * sizeof(float) : 0;
    const bool wide = width % 4 == 0 && reinterpret_cast<uintptr_t>(h) % 16 == 0;
#define MLR_GO(TO, S, V)                                                                                                                   \
    do {                                                                                                                                   \
        if (shared > 48 * 1024)                                                                                                            \
            cudaFuncSetAttribute(streams_step_kernel<TO, S, V>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(shared));    \
        mlr_launch((streams_step_kernel<TO, S, V>), dim3(count), dim3(kThreads), shared, stream, h, y, ld_y, y_scale, mix, w_out, w_in,    \
                   norm_weight, eps, static_cast<TO*>(out), ld_out, rows, width, streams);                                                 \
    } while (0)
#define MLR_PICK(TO, S)                  \
    do {                                 \
        if (wide) MLR_GO(TO, S, 4);      \
        else MLR_GO(TO, S, 1);           \
    } while (0)
#define MLR_COPIES(TO)                                     \
    switch (streams) {                                     \
        case 1: MLR_PICK(TO, 1); break;                    \
        case 2: MLR_PICK(TO, 2); break;                    \
        case 3: MLR_PICK(TO, 3); break;                    \
        case 4: MLR_PICK(TO, 4); break;                    \
        case 5: MLR_PICK(TO, 5); break;                    \
        case 6: MLR_PICK(TO, 6); break;                    \
        case 7: MLR_PICK(TO, 7); break;                    \
        case 8: MLR_PICK(TO, 8); break;                    \
        default: MLR_GO(TO, 0, 1); break;                  \
    }
    if (out_bf16) { MLR_COPIES(__nv_bfloat16) } else { MLR_COPIES(float) }
#undef MLR_COPIES
#undef MLR_PICK
#undef MLR_GO
    return mlr_launched("streams_step");
}

// pairs: [buckets + 1, width] or null (then no state is touched).  state: int32, one value per request slot, `state_stride` apart.
MLR_API int mlr_embed_hashed(float* h, const void* table, const void* pairs, int table_bf16, const int* ids, const int* segment_of_row,
                             const int* segment_info, int* state, long long state_stride, int rows, int width, int vocab, int streams,
                             float scale, int buckets, int mul_prev, int mul_cur, int* status, cudaStream_t stream) {
    MLR_REQUIRE(h && table && ids && width > 0 && vocab > 0 && streams >= 1 && streams <= kMaxStreams, "embed_hashed: bad arguments");
    MLR_REQUIRE(!pairs || (buckets > 0 && state && segment_of_row && segment_info), "embed_hashed: a table of pairs needs its size and the state");
    if (rows <= 0) return 0;
    if (table_bf16)
        mlr_launch((embed_hashed_kernel<__nv_bfloat16>), dim3(rows), dim3(kThreads), 0, stream, h, static_cast<const __nv_bfloat16*>(table),
                   static_cast<const __nv_bfloat16*>(pairs), ids, segment_of_row, segment_info, state, state_stride, width, vocab, streams, scale,
                   buckets, mul_prev, mul_cur, status);
    else
        mlr_launch((embed_hashed_kernel<float>), dim3(rows), dim3(kThreads), 0, stream, h, static_cast<const float*>(table),
                   static_cast<const float*>(pairs), ids, segment_of_row, segment_info, state, state_stride, width, vocab, streams, scale, buckets,
                   mul_prev, mul_cur, status);
    return mlr_launched("embed_hashed");
}
