// Attention over a paged cache whose keys and values may differ in size, with the pieces that
// vary between designs as parameters of one description (`MaskedAttentionSpec`, host memory):
//
//   which keys a query at position p sees:   j <= p,  j > p - window (window > 0),
//                                             j >= floor(p / chunk) * chunk (chunk > 0: chunks are
//                                             counted from position 0 of the sequence)
//   rotation:   the first rot_dims values of each head of q and k turned by p * freq[i], value i paired
//               with value i + rot_dims / 2; the rest pass.  Angles, cosines and sines are float32 and
//               computed from the position (no table, no largest position).
//   sink:       softmax with exp(0) added to the denominator (a key of score 0 without a value)
//   gate:       out *= sigmoid(gate) or silu(gate), element by element, and a constant factor
//
// Cache of a layer: per page, the keys [kv_head][token_in_page][dim] and then the values
// [kv_head][token_in_page][vdim].  `mlr_kv_rope_cache` rotates the step's keys and writes keys and
// values; `mlr_attention_masked` rotates its query as it loads it and walks the visible keys in tiles
// of 64 with a running maximum, one block per (row, query head), so a row's result depends on its
// position and on the cache only.  Scores, weights and sums are float32; q, the cache, the gate and
// the output are float32 or bfloat16.  Keys that are not visible are never loaded.
#include "common.cuh"

struct MaskedAttentionSpec {
    const float* freq;     // [rot_dims / 2] float32 on the device, or null
    int heads, kv_heads, dim, vdim;
    int rot_dims, window, chunk, sink;
    int gate_kind;         // 0 none, 1 sigmoid, 2 silu
    float scale, out_scale;
};

namespace {

constexpr int kTile = 64;
constexpr int kThreads = 128;
constexpr int kMaxDimsPerThread = 2;  // vdim <= 256

template <typename T>
__global__ void __launch_bounds__(kThreads) kv_rope_cache_kernel(const T* k, int ld_k, const T* v, int ld_v, T* cache, int num_pages,
                                                                 const int* positions, const int* segment_of_row,
                                                                 const int* block_table, int table_stride, int page_size,
                                                                 MaskedAttentionSpec s, int* status) {
    mlr_grid_dependents_may_start();
    mlr_grid_wait();
    const int row = blockIdx.x;
    const int position = positions[row];
    const int page = block_table[static_cast<size_t>(segment_of_row[row]) * table_stride + position / page_size];
    if (page < 0 || page >= num_pages) {
        if (threadIdx.x == 0 && status) atomicOr(status, MLR_STATUS_BAD_PAGE);
        return;
    }
    const size_t page_elems = static_cast<size_t>(s.kv_heads) * page_size * (s.dim + s.vdim);
    T* kbase = cache + page * page_elems + static_cast<size_t>(position % page_size) * s.dim;
    T* vbase = cache + page * page_elems + static_cast<size_t>(s.kv_heads) * page_size * s.dim +
               static_cast<size_t>(position % page_size) * s.vdim;
    const T* krow = k + static_cast<size_t>(row) * ld_k;
    const T* vrow = v + static_cast<size_t>(row) * ld_v;
    const int half = s.rot_dims / 2;
    const float p = static_cast<float>(position);
    for (int i = threadIdx.x; i < s.kv_heads * s.dim; i += kThreads) {
        const int head = i / s.dim, c = i % s.dim;
        float value = mlr_load(krow, i);
        if (c < s.rot_dims) {
            float sn, cs;
            sincosf(p * s.freq[c < half ? c : c - half], &sn, &cs);
            const float other = mlr_load(krow, c < half ? i + half : i - half);
            value = c < half ? value * cs - other * sn : value * cs + other * sn;
        }
        mlr_store(kbase + static_cast<size_t>(head) * page_size * s.dim, c, value);
    }
    for (int i = threadIdx.x; i < s.kv_heads * s.vdim; i += kThreads) {
        const int head = i / s.vdim, c = i % s.vdim;
        vbase[static_cast<size_t>(head) * page_size * s.vdim + c] = vrow[i];
    }
}

template <typename T>
__global__ void __launch_bounds__(kThreads) attention_masked_kernel(const T* q, int ldq, const T* gate, int ld_gate, T* out, int ldo,
                                                                    const T* cache, int num_pages, const int* positions,
                                                                    const int* segment_of_row, const int* block_table,
                                                                    int table_stride, int page_size, MaskedAttentionSpec s,
                                                                    int* status) {
    mlr_grid_dependents_may_start();
    mlr_grid_wait();
    extern __shared__ __align__(16) unsigned char smem[];
    long long* offsets = reinterpret_cast<long long*>(smem);   // [kTile] element offset of the token's value row
    float* scores = reinterpret_cast<float*>(offsets + kTile);  // [kTile]
    float* qs = scores + kTile;                                  // [dim]
    __shared__ int bad;

    const int row = blockIdx.x, head = blockIdx.y;
    const int kv_head = head / (s.heads / s.kv_heads);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int position = positions[row];
    const int segment = segment_of_row[row];
    int lo = 0;
    if (s.window > 0) lo = max(lo, position - s.window + 1);
    if (s.chunk > 0) lo = max(lo, (position / s.chunk) * s.chunk);
    const int* table = block_table + static_cast<size_t>(segment) * table_stride;
    const size_t page_elems = static_cast<size_t>(s.kv_heads) * page_size * (s.dim + s.vdim);
    const size_t key_plane = static_cast<size_t>(s.kv_heads) * page_size * s.dim;

    const T* qrow = q + static_cast<size_t>(row) * ldq + static_cast<size_t>(head) * s.dim;
    const int half = s.rot_dims / 2;
    const float p = static_cast<float>(position);
    for (int c = threadIdx.x; c < s.dim; c += kThreads) {
        float value = mlr_load(qrow, c);
        if (c < s.rot_dims) {
            float sn, cs;
            sincosf(p * s.freq[c < half ? c : c - half], &sn, &cs);
            const float other = mlr_load(qrow, c < half ? c + half : c - half);
            value = c < half ? value * cs - other * sn : value * cs + other * sn;
        }
        qs[c] = value;
    }
    if (threadIdx.x == 0) bad = 0;
    __syncthreads();

    // The sink is a key of score 0 that is always seen and carries no value.
    float running_max = s.sink ? 0.0f : -INFINITY, running_sum = s.sink ? 1.0f : 0.0f;
    float acc[kMaxDimsPerThread] = {0.0f, 0.0f};

    for (int tile = (lo / kTile) * kTile; tile <= position; tile += kTile) {
        for (int i = warp; i < kTile; i += kThreads / 32) {
            const int t = tile + i;
            float score = -INFINITY;
            long long offset = -1;
            if (t >= lo && t <= position) {
                const int page = table[t / page_size];
                if (page < 0 || page >= num_pages) {
                    if (lane == 0) bad = 1;
                } else {
                    const T* k = cache + page * page_elems + (static_cast<size_t>(kv_head) * page_size + t % page_size) * s.dim;
                    offset = static_cast<long long>(page * page_elems + key_plane +
                                                    (static_cast<size_t>(kv_head) * page_size + t % page_size) * s.vdim);
                    float partial = 0.0f;
                    for (int j = lane; j < s.dim; j += 32) partial = fmaf(qs[j], mlr_load(k, j), partial);
                    score = mlr_warp_sum(partial) * s.scale;
                }
            }
            if (lane == 0) {
                scores[i] = score;
                offsets[i] = offset;
            }
        }
        __syncthreads();
        float tile_max = -INFINITY;
        for (int i = 0; i < kTile; ++i) tile_max = fmaxf(tile_max, scores[i]);
        const float new_max = fmaxf(running_max, tile_max);
        __syncthreads();
        if (threadIdx.x < kTile) {
            const float sc = scores[threadIdx.x];
            scores[threadIdx.x] = (sc == -INFINITY) ? 0.0f : expf(sc - new_max);
        }
        __syncthreads();
        if (new_max > -INFINITY) {
            const float alpha = running_max == -INFINITY ? 0.0f : expf(running_max - new_max);
            running_sum *= alpha;
#pragma unroll
            for (int d = 0; d < kMaxDimsPerThread; ++d) acc[d] *= alpha;
            for (int i = 0; i < kTile; ++i) {
                const long long offset = offsets[i];
                if (offset < 0) continue;
                const float w = scores[i];
                running_sum += w;
                const T* v = cache + offset;
#pragma unroll
                for (int d = 0; d < kMaxDimsPerThread; ++d) {
                    const int c = threadIdx.x + d * kThreads;
                    if (c < s.vdim) acc[d] = fmaf(w, mlr_load(v, c), acc[d]);
                }
            }
            running_max = new_max;
        }
        __syncthreads();
    }
    if (bad && threadIdx.x == 0 && status) atomicOr(status, MLR_STATUS_BAD_PAGE);
    T* orow = out + static_cast<size_t>(row) * ldo + static_cast<size_t>(head) * s.vdim;
    const T* grow = gate ? gate + static_cast<size_t>(row) * ld_gate + static_cast<size_t>(head) * s.vdim : nullptr;
#pragma unroll
    for (int d = 0; d < kMaxDimsPerThread; ++d) {
        const int c = threadIdx.x + d * kThreads;
        if (c < s.vdim) {
            float value = running_sum > 0.0f ? acc[d] / running_sum : 0.0f;
            if (grow) {
                const float g = mlr_load(grow, c);
                const float sig = 1.0f / (1.0f + expf(-g));
                value *= s.gate_kind == 2 ? g * sig : sig;
            }
            mlr_store(orow, c, value * s.out_scale);
        }
    }
}

int check_spec(const MaskedAttentionSpec* s, const char* who) {
    MLR_REQUIRE(s, "%s: no description", who);
    MLR_REQUIRE(s->heads > 0 && s->kv_heads > 0 && s->heads % s->kv_heads == 0, "%s: %d query heads cannot share %d kv heads", who,
                s->heads, s->kv_heads);
    MLR_REQUIRE(s->dim >= 1 && s->dim <= 1024 && s->vdim >= 1 && s->vdim <= kThreads * kMaxDimsPerThread,
                "%s: key size %d or value size %d is outside what the kernel takes (1024, %d)", who, s->dim, s->vdim,
                kThreads * kMaxDimsPerThread);
    MLR_REQUIRE(s->rot_dims >= 0 && s->rot_dims % 2 == 0 && s->rot_dims <= s->dim && (s->rot_dims == 0 || s->freq),
                "%s: %d rotated values do not fit a head of %d (or no frequencies were given)", who, s->rot_dims, s->dim);
    MLR_REQUIRE(s->window >= 0 && s->chunk >= 0 && s->heads <= 65535, "%s: bad window, chunk or head count", who);
    return 0;
}

}  // namespace

MLR_API int mlr_kv_rope_cache(const MaskedAttentionSpec* spec, const void* k, int ld_k, const void* v, int ld_v, int act_bf16,
                              void* cache, int num_pages, const int* positions, const int* segment_of_row, const int* block_table,
                              int table_stride, int page_size, int rows, int* status, cudaStream_t stream) {
    if (check_spec(spec, "kv_rope_cache")) return 1;
    MLR_REQUIRE(rows >= 0 && page_size > 0 && num_pages > 0 && cache && block_table, "kv_rope_cache: bad sizes or no cache");
    MLR_REQUIRE(ld_k >= spec->kv_heads * spec->dim && ld_v >= spec->kv_heads * spec->vdim, "kv_rope_cache: a row stride is smaller than the row");
    if (rows == 0) return 0;
    if (act_bf16)
        mlr_launch((kv_rope_cache_kernel<__nv_bfloat16>), dim3(rows), dim3(kThreads), 0, stream, static_cast<const __nv_bfloat16*>(k), ld_k,
                   static_cast<const __nv_bfloat16*>(v), ld_v, static_cast<__nv_bfloat16*>(cache), num_pages, positions, segment_of_row,
                   block_table, table_stride, page_size, *spec, status);
    else
        mlr_launch((kv_rope_cache_kernel<float>), dim3(rows), dim3(kThreads), 0, stream, static_cast<const float*>(k), ld_k,
                   static_cast<const float*>(v), ld_v, static_cast<float*>(cache), num_pages, positions, segment_of_row, block_table,
                   table_stride, page_size, *spec, status);
    return mlr_launched("kv_rope_cache");
}

MLR_API int mlr_attention_masked(const MaskedAttentionSpec* spec, const void* q, int ldq, const void* gate, int ld_gate, void* out,
                                 int ldo, int act_bf16, const void* cache, int num_pages, const int* positions,
                                 const int* segment_of_row, const int* block_table, int table_stride, int page_size, int rows,
                                 int* status, cudaStream_t stream) {
    if (check_spec(spec, "attention_masked")) return 1;
    MLR_REQUIRE(rows >= 0 && page_size > 0 && num_pages > 0, "attention_masked: bad page size or page count");
    MLR_REQUIRE(ldq >= spec->heads * spec->dim && ldo >= spec->heads * spec->vdim, "attention_masked: a row stride is smaller than the row");
    MLR_REQUIRE((spec->gate_kind == 0) == (gate == nullptr), "attention_masked: the description and the call disagree about a gate");
    if (rows == 0) return 0;
    const size_t shared = sizeof(float) * (spec->dim + kTile) + sizeof(long long) * kTile + 16;
    const dim3 grid(rows, spec->heads);
    if (act_bf16)
        mlr_launch((attention_masked_kernel<__nv_bfloat16>), dim3(grid), dim3(kThreads), shared, stream,
                   static_cast<const __nv_bfloat16*>(q), ldq, static_cast<const __nv_bfloat16*>(gate), ld_gate,
                   static_cast<__nv_bfloat16*>(out), ldo, static_cast<const __nv_bfloat16*>(cache), num_pages, positions, segment_of_row,
                   block_table, table_stride, page_size, *spec, status);
    else
        mlr_launch((attention_masked_kernel<float>), dim3(grid), dim3(kThreads), shared, stream, static_cast<const float*>(q), ldq,
                   static_cast<const float*>(gate), ld_gate, static_cast<float*>(out), ldo, static_cast<const float*>(cache), num_pages,
                   positions, segment_of_row, block_table, table_stride, page_size, *spec, status);
    return mlr_launched("attention_masked");
}
