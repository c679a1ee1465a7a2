// Mixers that keep a matrix per head and request instead of keys and values: a state S [dim, vdim],
// float32, that every token updates and reads.  One kernel serves the family; what varies between
// designs is a description in host memory (`RecurrenceSpec`):
//
//   activation of q, k and v as they are loaded (in_act): none, or SiLU
//   preparation of q and k (float32, from the projections' output):
//       rotate:  the first rot_dims values turned by position * freq[i] (value i paired with i + rot_dims/2)
//       unit:    x / sqrt(sum(x^2) + unit_eps)
//     then q *= q_mult, k *= k_mult
//   rule, token by token:
//       decay:   S <- decay[head] S + k v^T;                            o = S^T q       (retention)
//       delta:   S <- g S;  u = beta (v - S^T k);  S <- S + k u^T;      o = S^T q       (gated delta rule)
//                with g = exp(-exp(a_log[head]) softplus(a + dt_bias[head])), beta = sigmoid(b), from two more
//                columns of the projections' output per head
//   (q, k, v come from one buffer, `proj`; a, b and the gate from another, `side`, which may be the same)
//   read-out:    o / sqrt(mean(o^2) + eps) per head, times a weight [vdim] (optional), times silu(gate)
//                or sigmoid(gate) (optional), times a constant; with norm_all the root mean square is taken over
//                the outputs of all heads of a token together and the weight is [heads * vdim]
//
// The columns of S are independent of one another in both rules, so a warp owns a few columns (lanes
// split `dim`), and one block owns one (request, head): it prepares a batch of tokens in shared memory,
// its warps walk the batch token by token, and the block norms and gates the batch's outputs.  The
// state is read at the start and written at the end; a new request's state is zero (the caller zeroes
// the slot).  Everything but the loads of the projections and the store of the result is float32.
//
// `mlr_short_conv` is the causal convolution over time per channel that precedes such a mixer in some
// designs (taps [channels, n], the last tap is the current token's; silu after it), with the last n-1
// inputs of every request kept as state; `mlr_short_conv_state` moves that state on after a step.
#include "common.cuh"

#include <type_traits>

struct RecurrenceSpec {
    const float* freq;         // [rot_dims / 2] or null
    const float* decay;        // [heads] (rule 0)
    const float* a_log;        // [heads] (rule 1)
    const float* dt_bias;      // [heads] (rule 1)
    const float* out_weight;   // [vdim] or null
    int heads, qk_heads, dim, vdim;
    int prep;                  // 0 none, 1 rotate, 2 unit
    int rot_dims;
    int rule;                  // 0 decay, 1 delta
    int gate_kind;             // 0 none, 1 sigmoid, 2 silu
    int col_q, col_k, col_v;           // first columns of q, k, v in `proj`
    int col_a, col_b, col_gate;        // first columns of the rule's two inputs and of the gate in `side`
    int in_act;                        // 0: q, k, v as projected; 1: through SiLU
    int norm_all;                      // 0: the read-out norms every head alone; 1: all heads of a token together
    float q_mult, k_mult, unit_eps, eps, out_scale;
};

namespace {

__device__ __forceinline__ float softplus(float x) { return x > 20.0f ? x : log1pf(expf(x)); }
__device__ __forceinline__ float act_in(float x, int kind) { return kind == 1 ? x / (1.0f + expf(-x)) : x; }
// The turn of a pair by an angle, with its roundings spelled out: the one-kernel form and the prepare kernel give the same bits.
__device__ __forceinline__ void turn(float u, float v, float cs, float sn, float& a, float& b) {
    a = __fmaf_rn(u, cs, -__fmul_rn(v, sn));
    b = __fmaf_rn(v, cs, __fmul_rn(u, sn));
}

template <typename T, int R, int COLS>
__global__ void __launch_bounds__(1024) linear_recurrence_kernel(const T* proj, int ld, const T* side, int ld_side, T* out, int ld_out, float* state,
                                                                  long long state_stride, const int* segment_info, RecurrenceSpec s,
                                                                  int batch, float* raw) {
    mlr_grid_wait();
    extern __shared__ __align__(16) unsigned char smem[];
    float* qs = reinterpret_cast<float*>(smem);          // [batch][dim]
    float* ks = qs + static_cast<size_t>(batch) * s.dim; // [batch][dim]
    float* vs = ks + static_cast<size_t>(batch) * s.dim; // [batch][vdim]
    float* os = vs + static_cast<size_t>(batch) * s.vdim;  // [batch][vdim]
    float* gs = os + static_cast<size_t>(batch) * s.vdim;  // [batch]
    float* bs = gs + batch;                                 // [batch]

    const int segment = blockIdx.x, head = blockIdx.y;
    const int first = segment_info[4 * segment], count = segment_info[4 * segment + 1];
    const int start = segment_info[4 * segment + 2], slot = segment_info[4 * segment + 3];
    const int qk_head = head / (s.heads / s.qk_heads);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    const int threads = blockDim.x;
    const int col0 = warp * COLS;

    float S[COLS][R];
    float* my_state = state + static_cast<size_t>(slot) * state_stride + (static_cast<size_t>(head) * s.vdim) * s.dim;
#pragma unroll
    for (int c = 0; c < COLS; ++c)
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const int d = lane + 32 * r;
            S[c][r] = (col0 + c < s.vdim && d < s.dim) ? my_state[static_cast<size_t>(col0 + c) * s.dim + d] : 0.0f;
        }
    const float decay = s.rule == 0 ? s.decay[head] : 1.0f;
    const int half = s.rot_dims / 2;

    for (int base = 0; base < count; base += batch) {
        const int n = min(batch, count - base);
        // ---- prepare the batch: q, k, v (and the gates of the rule) as float32
        for (int i = threadIdx.x; i < n * s.dim; i += threads) {
            const int t = i / s.dim, c = i % s.dim;
            const T* row = proj + static_cast<size_t>(first + base + t) * ld;
            qs[i] = act_in(mlr_load(row, s.col_q + qk_head * s.dim + c), s.in_act);
            ks[i] = act_in(mlr_load(row, s.col_k + qk_head * s.dim + c), s.in_act);
        }
        for (int i = threadIdx.x; i < n * s.vdim; i += threads) {
            const int t = i / s.vdim, c = i % s.vdim;
            vs[i] = act_in(mlr_load(proj + static_cast<size_t>(first + base + t) * ld, s.col_v + head * s.vdim + c), s.in_act);
        }
        if (s.rule == 1 && threadIdx.x < n) {
            const T* row = side + static_cast<size_t>(first + base + threadIdx.x) * ld_side;
            const float a = mlr_load(row, s.col_a + head), b = mlr_load(row, s.col_b + head);
            gs[threadIdx.x] = expf(-expf(s.a_log[head]) * softplus(a + s.dt_bias[head]));
            bs[threadIdx.x] = 1.0f / (1.0f + expf(-b));
        }
        __syncthreads();
        if (s.prep == 1) {
            for (int i = threadIdx.x; i < n * half; i += threads) {
                const int t = i / half, c = i % half;
                float sn, cs;
                sincosf(static_cast<float>(start + base + t) * s.freq[c], &sn, &cs);
                float* x = qs + static_cast<size_t>(t) * s.dim;
                turn(x[c], x[c + half], cs, sn, x[c], x[c + half]);
                x = ks + static_cast<size_t>(t) * s.dim;
                turn(x[c], x[c + half], cs, sn, x[c], x[c + half]);
            }
            __syncthreads();
            for (int i = threadIdx.x; i < n * s.dim; i += threads) {
                qs[i] = __fmul_rn(qs[i], s.q_mult);
                ks[i] = __fmul_rn(ks[i], s.k_mult);
            }
        } else if (s.prep == 2) {
            for (int vec = warp; vec < 2 * n; vec += warps) {
                float* x = (vec < n ? qs : ks) + static_cast<size_t>(vec < n ? vec : vec - n) * s.dim;
                float sum = 0.0f;
                for (int c = lane; c < s.dim; c += 32) sum = fmaf(x[c], x[c], sum);
                const float inv = 1.0f / sqrtf(mlr_warp_sum(sum) + s.unit_eps);
                const float mult = vec < n ? s.q_mult : s.k_mult;
                for (int c = lane; c < s.dim; c += 32) x[c] = x[c] * inv * mult;
            }
        } else {
            for (int i = threadIdx.x; i < n * s.dim; i += threads) {
                qs[i] *= s.q_mult;
                ks[i] *= s.k_mult;
            }
        }
        __syncthreads();
        // ---- the recurrence: this warp's columns, token by token
        if (col0 < s.vdim) {
            for (int t = 0; t < n; ++t) {
                float kk[R], qq[R];
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    const int d = lane + 32 * r;
                    kk[r] = d < s.dim ? ks[static_cast<size_t>(t) * s.dim + d] : 0.0f;
                    qq[r] = d < s.dim ? qs[static_cast<size_t>(t) * s.dim + d] : 0.0f;
                }
                float o[COLS];
                if (s.rule == 0) {
#pragma unroll
                    for (int c = 0; c < COLS; ++c) {
                        const float v = col0 + c < s.vdim ? vs[static_cast<size_t>(t) * s.vdim + col0 + c] : 0.0f;
                        float dot = 0.0f;
#pragma unroll
                        for (int r = 0; r < R; ++r) {
                            S[c][r] = fmaf(decay, S[c][r], kk[r] * v);
                            dot = fmaf(S[c][r], qq[r], dot);
                        }
                        o[c] = dot;
                    }
                } else {
                    const float g = gs[t], beta = bs[t];
                    float dotk[COLS];
#pragma unroll
                    for (int c = 0; c < COLS; ++c) {
                        float dot = 0.0f;
#pragma unroll
                        for (int r = 0; r < R; ++r) {
                            S[c][r] *= g;
                            dot = fmaf(S[c][r], kk[r], dot);
                        }
                        dotk[c] = dot;
                    }
#pragma unroll
                    for (int c = 0; c < COLS; ++c) dotk[c] = mlr_warp_sum(dotk[c]);
#pragma unroll
                    for (int c = 0; c < COLS; ++c) {
                        const float v = col0 + c < s.vdim ? vs[static_cast<size_t>(t) * s.vdim + col0 + c] : 0.0f;
                        const float u = beta * (v - dotk[c]);
                        float dot = 0.0f;
#pragma unroll
                        for (int r = 0; r < R; ++r) {
                            S[c][r] = fmaf(kk[r], u, S[c][r]);
                            dot = fmaf(S[c][r], qq[r], dot);
                        }
                        o[c] = dot;
                    }
                }
#pragma unroll
                for (int c = 0; c < COLS; ++c) o[c] = mlr_warp_sum(o[c]);
                if (lane == 0) {
#pragma unroll
                    for (int c = 0; c < COLS; ++c)
                        if (col0 + c < s.vdim) os[static_cast<size_t>(t) * s.vdim + col0 + c] = o[c];
                }
            }
        }
        __syncthreads();
        // ---- read-out of the batch: norm per head, weight, gate; or the plain float32 outputs for a read-out kernel
        for (int t = warp; t < n; t += warps) {
            const float* o = os + static_cast<size_t>(t) * s.vdim;
            if (raw) {
                float* rrow = raw + (static_cast<size_t>(first + base + t) * s.heads + head) * s.vdim;
                for (int c = lane; c < s.vdim; c += 32) rrow[c] = o[c];
                continue;
            }
            float inv = 1.0f;
            if (s.eps >= 0.0f) {
                float sum = 0.0f;
                for (int c = lane; c < s.vdim; c += 32) sum = fmaf(o[c], o[c], sum);
                inv = 1.0f / sqrtf(mlr_warp_sum(sum) / static_cast<float>(s.vdim) + s.eps);
            }
            const T* prow = side + static_cast<size_t>(first + base + t) * ld_side;
            T* orow = out + static_cast<size_t>(first + base + t) * ld_out + static_cast<size_t>(head) * s.vdim;
            for (int c = lane; c < s.vdim; c += 32) {
                float value = o[c] * inv;
                if (s.out_weight) value *= s.out_weight[c];
                if (s.gate_kind) {
                    const float g = mlr_load(prow, s.col_gate + head * s.vdim + c);
                    const float sig = 1.0f / (1.0f + expf(-g));
                    value *= s.gate_kind == 2 ? g * sig : sig;
                }
                mlr_store(orow, c, value * s.out_scale);
            }
        }
        __syncthreads();
    }
    mlr_grid_dependents_may_start();
#pragma unroll
    for (int c = 0; c < COLS; ++c)
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const int d = lane + 32 * r;
            if (col0 + c < s.vdim && d < s.dim) my_state[static_cast<size_t>(col0 + c) * s.dim + d] = S[c][r];
        }
}

// ---- the same in three kernels, for steps of many rows.  The fused kernel above has one block per (request, head):
// a long prompt of one request then runs on a handful of SMs, and every block prepares q and k itself.  Here the
// preparation and the read-out are parallel over rows, and the scan, the only sequential part, has a block per
// (request, head, group of 16 columns of the state).

// q and k of every row, prepared, as float32 [rows, qk_heads * dim] each; for the delta rule also g and beta [rows, 2 * heads].
template <typename T>
__global__ void __launch_bounds__(128) recurrence_prepare_kernel(const T* proj, int ld, const T* side, int ld_side, float* qf, float* kf,
                                                                 float* gates, const int* positions, RecurrenceSpec s) {
    mlr_grid_wait();
    const int row = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    const T* in = proj + static_cast<size_t>(row) * ld;
    const float position = static_cast<float>(positions[row]);
    const int half = s.rot_dims / 2;
    const size_t out_ld = static_cast<size_t>(s.qk_heads) * s.dim;
    for (int vec = warp; vec < 2 * s.qk_heads; vec += warps) {
        const bool is_q = vec < s.qk_heads;
        const int head = is_q ? vec : vec - s.qk_heads;
        const T* x = in + (is_q ? s.col_q : s.col_k) + head * s.dim;
        float* y = (is_q ? qf : kf) + row * out_ld + static_cast<size_t>(head) * s.dim;
        const float mult = is_q ? s.q_mult : s.k_mult;
        if (s.prep == 1) {
            for (int c = lane; c < half; c += 32) {
                float sn, cs;
                sincosf(position * s.freq[c], &sn, &cs);
                const float u = act_in(mlr_load(x, c), s.in_act), v = act_in(mlr_load(x, c + half), s.in_act);
                float a, b;
                turn(u, v, cs, sn, a, b);
                y[c] = __fmul_rn(a, mult);
                y[c + half] = __fmul_rn(b, mult);
            }
            for (int c = s.rot_dims + lane; c < s.dim; c += 32) y[c] = act_in(mlr_load(x, c), s.in_act) * mult;
        } else if (s.prep == 2) {
            float sum = 0.0f;
            for (int c = lane; c < s.dim; c += 32) {
                const float v = act_in(mlr_load(x, c), s.in_act);
                sum = fmaf(v, v, sum);
            }
            const float inv = 1.0f / sqrtf(mlr_warp_sum(sum) + s.unit_eps);
            for (int c = lane; c < s.dim; c += 32) y[c] = act_in(mlr_load(x, c), s.in_act) * inv * mult;
        } else {
            for (int c = lane; c < s.dim; c += 32) y[c] = act_in(mlr_load(x, c), s.in_act) * mult;
        }
    }
    if (s.rule == 1) {
        const T* sd = side + static_cast<size_t>(row) * ld_side;
        for (int h = threadIdx.x; h < s.heads; h += blockDim.x) {
            const float a = mlr_load(sd, s.col_a + h), b = mlr_load(sd, s.col_b + h);
            gates[static_cast<size_t>(row) * 2 * s.heads + h] = expf(-expf(s.a_log[h]) * softplus(a + s.dt_bias[h]));
            gates[static_cast<size_t>(row) * 2 * s.heads + s.heads + h] = 1.0f / (1.0f + expf(-b));
        }
    }
    mlr_grid_dependents_may_start();
}

constexpr int kScanWarps = 4, kScanCols = 4, kScanBlockCols = kScanWarps * kScanCols;

template <typename T, int R>
__global__ void __launch_bounds__(kScanWarps * 32) recurrence_scan_kernel(const float* qf, const float* kf, const float* gates, const T* proj,
                                                                          int ld, float* obuf, float* state, long long state_stride,
                                                                          const int* segment_info, RecurrenceSpec s, int batch) {
    mlr_grid_wait();
    extern __shared__ __align__(16) unsigned char smem[];
    const size_t stage = static_cast<size_t>(batch) * s.dim;
    float* qs = reinterpret_cast<float*>(smem);                // [2][batch][dim]: a batch is copied while the one before is walked
    float* ks = qs + 2 * stage;                                // [2][batch][dim]
    float* vs = ks + 2 * stage;                                // [batch][16]
    float* os = vs + static_cast<size_t>(batch) * kScanBlockCols;   // [batch][16]
    float* gs = os + static_cast<size_t>(batch) * kScanBlockCols;   // [batch]
    float* bs = gs + batch;                                    // [batch]
    const int segment = blockIdx.x, head = blockIdx.y, block_col = blockIdx.z * kScanBlockCols;
    const int first = segment_info[4 * segment], count = segment_info[4 * segment + 1], slot = segment_info[4 * segment + 3];
    const int qk_head = head / (s.heads / s.qk_heads);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int col0 = block_col + warp * kScanCols;
    const size_t qk_ld = static_cast<size_t>(s.qk_heads) * s.dim;
    const size_t o_ld = static_cast<size_t>(s.heads) * s.vdim;
    const bool wide = s.dim % 4 == 0;                          // rows of q and k start on 16-byte borders

    float S[kScanCols][R];
    float* my_state = state + static_cast<size_t>(slot) * state_stride + (static_cast<size_t>(head) * s.vdim) * s.dim;
#pragma unroll
    for (int c = 0; c < kScanCols; ++c)
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const int d = lane + 32 * r;
            S[c][r] = (col0 + c < s.vdim && d < s.dim) ? my_state[static_cast<size_t>(col0 + c) * s.dim + d] : 0.0f;
        }
    const float decay = s.rule == 0 ? s.decay[head] : 1.0f;

    constexpr int kVPerThread = 32 * kScanBlockCols / (kScanWarps * 32);     // batch <= 32
    float v_next[kVPerThread], g_next = 0.0f, b_next = 0.0f;
    // Starts the copies of a batch's q and k into a stage and loads its v, g and beta into registers.
    auto fetch = [&](int base, int into) {
        const int n = min(batch, count - base);
        const float* qsrc = qf + static_cast<size_t>(first + base) * qk_ld + static_cast<size_t>(qk_head) * s.dim;
        const float* ksrc = kf + static_cast<size_t>(first + base) * qk_ld + static_cast<size_t>(qk_head) * s.dim;
        float* qdst = qs + into * stage;
        float* kdst = ks + into * stage;
        if (wide) {
            const int per_row = s.dim / 4;
            for (int i = threadIdx.x; i < n * per_row; i += blockDim.x) {
                const int t = i / per_row, c = (i % per_row) * 4;
                mlr_async_copy16(qdst + static_cast<size_t>(t) * s.dim + c, qsrc + t * qk_ld + c);
                mlr_async_copy16(kdst + static_cast<size_t>(t) * s.dim + c, ksrc + t * qk_ld + c);
            }
        } else {
            for (int i = threadIdx.x; i < n * s.dim; i += blockDim.x) {
                const int t = i / s.dim, c = i % s.dim;
                mlr_async_copy4(qdst + static_cast<size_t>(t) * s.dim + c, qsrc + t * qk_ld + c);
                mlr_async_copy4(kdst + static_cast<size_t>(t) * s.dim + c, ksrc + t * qk_ld + c);
            }
        }
        mlr_async_commit();
#pragma unroll
        for (int j = 0; j < kVPerThread; ++j) {
            const int i = threadIdx.x + j * kScanWarps * 32;
            const int t = i / kScanBlockCols, c = block_col + i % kScanBlockCols;
            v_next[j] = (t < n && c < s.vdim) ? mlr_load(proj + static_cast<size_t>(first + base + t) * ld, s.col_v + head * s.vdim + c) : 0.0f;
        }
        if (s.rule == 1 && threadIdx.x < n) {
            g_next = __ldcg(gates + static_cast<size_t>(first + base + threadIdx.x) * 2 * s.heads + head);
            b_next = __ldcg(gates + static_cast<size_t>(first + base + threadIdx.x) * 2 * s.heads + s.heads + head);
        }
    };

    fetch(0, 0);
    int current = 0;
    for (int base = 0; base < count; base += batch, current ^= 1) {
        const int n = min(batch, count - base);
        __syncthreads();                    // the batch before has been walked and written out
#pragma unroll
        for (int j = 0; j < kVPerThread; ++j) {
            const int i = threadIdx.x + j * kScanWarps * 32;
            if (i < batch * kScanBlockCols) vs[i] = act_in(v_next[j], s.in_act);
        }
        if (threadIdx.x < batch) {
            gs[threadIdx.x] = g_next;
            bs[threadIdx.x] = b_next;
        }
        mlr_async_wait();
        __syncthreads();
        if (base + batch < count) fetch(base + batch, current ^ 1);
        const float* qnow = qs + current * stage;
        const float* know = ks + current * stage;
        for (int t = 0; t < n; ++t) {
            float kk[R], qq[R];
#pragma unroll
            for (int r = 0; r < R; ++r) {
                const int d = lane + 32 * r;
                kk[r] = d < s.dim ? know[static_cast<size_t>(t) * s.dim + d] : 0.0f;
                qq[r] = d < s.dim ? qnow[static_cast<size_t>(t) * s.dim + d] : 0.0f;
            }
            float o[kScanCols];
            if (s.rule == 0) {
#pragma unroll
                for (int c = 0; c < kScanCols; ++c) {
                    const float v = vs[t * kScanBlockCols + warp * kScanCols + c];
                    float dot = 0.0f;
#pragma unroll
                    for (int r = 0; r < R; ++r) {
                        S[c][r] = fmaf(decay, S[c][r], kk[r] * v);
                        dot = fmaf(S[c][r], qq[r], dot);
                    }
                    o[c] = dot;
                }
            } else {
                const float g = gs[t], beta = bs[t];
                float dotk[kScanCols];
#pragma unroll
                for (int c = 0; c < kScanCols; ++c) {
                    float dot = 0.0f;
#pragma unroll
                    for (int r = 0; r < R; ++r) {
                        S[c][r] *= g;
                        dot = fmaf(S[c][r], kk[r], dot);
                    }
                    dotk[c] = dot;
                }
#pragma unroll
                for (int c = 0; c < kScanCols; ++c) dotk[c] = mlr_warp_sum(dotk[c]);
#pragma unroll
                for (int c = 0; c < kScanCols; ++c) {
                    const float v = vs[t * kScanBlockCols + warp * kScanCols + c];
                    const float u = beta * (v - dotk[c]);
                    float dot = 0.0f;
#pragma unroll
                    for (int r = 0; r < R; ++r) {
                        S[c][r] = fmaf(kk[r], u, S[c][r]);
                        dot = fmaf(S[c][r], qq[r], dot);
                    }
                    o[c] = dot;
                }
            }
#pragma unroll
            for (int c = 0; c < kScanCols; ++c) o[c] = mlr_warp_sum(o[c]);
            if (lane == 0) {
#pragma unroll
                for (int c = 0; c < kScanCols; ++c) os[t * kScanBlockCols + warp * kScanCols + c] = o[c];
            }
        }
        __syncthreads();
        for (int i = threadIdx.x; i < n * kScanBlockCols; i += blockDim.x) {
            const int t = i / kScanBlockCols, c = block_col + i % kScanBlockCols;
            if (c < s.vdim) obuf[static_cast<size_t>(first + base + t) * o_ld + static_cast<size_t>(head) * s.vdim + c] = os[i];
        }
    }
    mlr_grid_dependents_may_start();     // only now: blocks of the next grid that wait on this SM slow the walk
#pragma unroll
    for (int c = 0; c < kScanCols; ++c)
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const int d = lane + 32 * r;
            if (col0 + c < s.vdim && d < s.dim) my_state[static_cast<size_t>(col0 + c) * s.dim + d] = S[c][r];
        }
}

// The same walk for head sizes that are a multiple of 32, with a warp's lanes as 4 columns x 8 lanes: a lane keeps E4 groups of
// four state values of ONE column (values 4 * (8 * e + lane % 8) + 0..3, so that the eight lanes of a column read 128
// consecutive bytes of k and q at a time), and a sum over a column is 3 exchanges among 8 lanes instead of 5 among 32.
template <typename T, int E4>
__global__ void __launch_bounds__(kScanWarps * 32) recurrence_scan8_kernel(const float* qf, const float* kf, const float* gates, const T* proj,
                                                                          int ld, float* obuf, float* state, long long state_stride,
                                                                          const int* segment_info, RecurrenceSpec s, int batch) {
    mlr_grid_wait();
    extern __shared__ __align__(16) unsigned char smem[];
    const size_t stage = static_cast<size_t>(batch) * s.dim;
    float* qs = reinterpret_cast<float*>(smem);                // [2][batch][dim]: a batch is copied while the one before is walked
    float* ks = qs + 2 * stage;                                // [2][batch][dim]
    float* vs = ks + 2 * stage;                                // [batch][16]
    float* os = vs + static_cast<size_t>(batch) * kScanBlockCols;   // [batch][16]
    float* gs = os + static_cast<size_t>(batch) * kScanBlockCols;   // [batch]
    float* bs = gs + batch;                                    // [batch]
    const int segment = blockIdx.x, head = blockIdx.y, block_col = blockIdx.z * kScanBlockCols;
    const int first = segment_info[4 * segment], count = segment_info[4 * segment + 1], slot = segment_info[4 * segment + 3];
    const int qk_head = head / (s.heads / s.qk_heads);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int col0 = block_col + warp * kScanCols;
    const size_t qk_ld = static_cast<size_t>(s.qk_heads) * s.dim;
    const size_t o_ld = static_cast<size_t>(s.heads) * s.vdim;
    const bool wide = s.dim % 4 == 0;                          // rows of q and k start on 16-byte borders

    const int sub = lane & 7, my_col = col0 + (lane >> 3);
    const bool live = my_col < s.vdim;
    float S[E4][4];
    float* my_state = state + static_cast<size_t>(slot) * state_stride + (static_cast<size_t>(head) * s.vdim) * s.dim;
#pragma unroll
    for (int e = 0; e < E4; ++e)
#pragma unroll
        for (int j = 0; j < 4; ++j) S[e][j] = live ? my_state[static_cast<size_t>(my_col) * s.dim + 4 * (8 * e + sub) + j] : 0.0f;
    const float decay = s.rule == 0 ? s.decay[head] : 1.0f;

    constexpr int kVPerThread = 32 * kScanBlockCols / (kScanWarps * 32);     // batch <= 32
    T v_next[kVPerThread];                // as loaded: a conversion right behind the load would wait for it
    float g_next = 0.0f, b_next = 0.0f;
    // Starts the copies of a batch's q and k into a stage and loads its v, g and beta into registers.
    auto fetch = [&](int base, int into) {
        const int n = min(batch, count - base);
        const float* qsrc = qf + static_cast<size_t>(first + base) * qk_ld + static_cast<size_t>(qk_head) * s.dim;
        const float* ksrc = kf + static_cast<size_t>(first + base) * qk_ld + static_cast<size_t>(qk_head) * s.dim;
        float* qdst = qs + into * stage;
        float* kdst = ks + into * stage;
        if (wide) {
            const int per_row = s.dim / 4;
            for (int i = threadIdx.x; i < n * per_row; i += blockDim.x) {
                const int t = i / per_row, c = (i % per_row) * 4;
                mlr_async_copy16(qdst + static_cast<size_t>(t) * s.dim + c, qsrc + t * qk_ld + c);
                mlr_async_copy16(kdst + static_cast<size_t>(t) * s.dim + c, ksrc + t * qk_ld + c);
            }
        } else {
            for (int i = threadIdx.x; i < n * s.dim; i += blockDim.x) {
                const int t = i / s.dim, c = i % s.dim;
                mlr_async_copy4(qdst + static_cast<size_t>(t) * s.dim + c, qsrc + t * qk_ld + c);
                mlr_async_copy4(kdst + static_cast<size_t>(t) * s.dim + c, ksrc + t * qk_ld + c);
            }
        }
        mlr_async_commit();
#pragma unroll
        for (int j = 0; j < kVPerThread; ++j) {
            const int i = threadIdx.x + j * kScanWarps * 32;
            const int t = i / kScanBlockCols, c = block_col + i % kScanBlockCols;
            v_next[j] = proj[(t < n && c < s.vdim) ? static_cast<size_t>(first + base + t) * ld + s.col_v + head * s.vdim + c : 0];
        }
        if (s.rule == 1 && threadIdx.x < n) {
            g_next = __ldcg(gates + static_cast<size_t>(first + base + threadIdx.x) * 2 * s.heads + head);
            b_next = __ldcg(gates + static_cast<size_t>(first + base + threadIdx.x) * 2 * s.heads + s.heads + head);
        }
    };

    fetch(0, 0);
    int current = 0;
    for (int base = 0; base < count; base += batch, current ^= 1) {
        const int n = min(batch, count - base);
        __syncthreads();                    // the batch before has been walked and written out
#pragma unroll
        for (int j = 0; j < kVPerThread; ++j) {
            const int i = threadIdx.x + j * kScanWarps * 32;
            if (i < batch * kScanBlockCols) vs[i] = act_in(mlr_load(&v_next[j], 0), s.in_act);
        }
        if (threadIdx.x < batch) {
            gs[threadIdx.x] = g_next;
            bs[threadIdx.x] = b_next;
        }
        mlr_async_wait();
        __syncthreads();
        if (base + batch < count) fetch(base + batch, current ^ 1);
        const float* qnow = qs + current * stage;
        const float* know = ks + current * stage;
        // Four tokens at a time: their sums over a column are exchanged together, and nothing is stored to shared
        // memory in between (a store there would keep the next token's loads from starting early).
        auto walk4 = [&](int t0, auto guarded) {
            float dots[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int t = t0 + u;
                dots[u] = 0.0f;
                if (!decltype(guarded)::value || t < n) {
                    const float4* k4 = reinterpret_cast<const float4*>(know + static_cast<size_t>(t) * s.dim);
                    const float4* q4 = reinterpret_cast<const float4*>(qnow + static_cast<size_t>(t) * s.dim);
                    float4 kk[E4], qq[E4];
#pragma unroll
                    for (int e = 0; e < E4; ++e) {
                        kk[e] = k4[8 * e + sub];
                        qq[e] = q4[8 * e + sub];
                    }
                    const float v = vs[t * kScanBlockCols + warp * kScanCols + (lane >> 3)];
                    float d0 = 0.0f, d1 = 0.0f, d2 = 0.0f, d3 = 0.0f;
                    if (s.rule == 0) {
#pragma unroll
                        for (int e = 0; e < E4; ++e) {
                            S[e][0] = fmaf(decay, S[e][0], kk[e].x * v); d0 = fmaf(S[e][0], qq[e].x, d0);
                            S[e][1] = fmaf(decay, S[e][1], kk[e].y * v); d1 = fmaf(S[e][1], qq[e].y, d1);
                            S[e][2] = fmaf(decay, S[e][2], kk[e].z * v); d2 = fmaf(S[e][2], qq[e].z, d2);
                            S[e][3] = fmaf(decay, S[e][3], kk[e].w * v); d3 = fmaf(S[e][3], qq[e].w, d3);
                        }
                    } else {
                        const float g = gs[t], beta = bs[t];
                        float c0 = 0.0f, c1 = 0.0f, c2 = 0.0f, c3 = 0.0f;
#pragma unroll
                        for (int e = 0; e < E4; ++e) {
                            S[e][0] *= g; c0 = fmaf(S[e][0], kk[e].x, c0);
                            S[e][1] *= g; c1 = fmaf(S[e][1], kk[e].y, c1);
                            S[e][2] *= g; c2 = fmaf(S[e][2], kk[e].z, c2);
                            S[e][3] *= g; c3 = fmaf(S[e][3], kk[e].w, c3);
                        }
                        float dk = (c0 + c1) + (c2 + c3);
                        dk += __shfl_xor_sync(0xffffffffu, dk, 1);
                        dk += __shfl_xor_sync(0xffffffffu, dk, 2);
                        dk += __shfl_xor_sync(0xffffffffu, dk, 4);
                        const float u_t = beta * (v - dk);
#pragma unroll
                        for (int e = 0; e < E4; ++e) {
                            S[e][0] = fmaf(kk[e].x, u_t, S[e][0]); d0 = fmaf(S[e][0], qq[e].x, d0);
                            S[e][1] = fmaf(kk[e].y, u_t, S[e][1]); d1 = fmaf(S[e][1], qq[e].y, d1);
                            S[e][2] = fmaf(kk[e].z, u_t, S[e][2]); d2 = fmaf(S[e][2], qq[e].z, d2);
                            S[e][3] = fmaf(kk[e].w, u_t, S[e][3]); d3 = fmaf(S[e][3], qq[e].w, d3);
                        }
                    }
                    dots[u] = (d0 + d1) + (d2 + d3);
                }
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) dots[u] += __shfl_xor_sync(0xffffffffu, dots[u], 1);
#pragma unroll
            for (int u = 0; u < 4; ++u) dots[u] += __shfl_xor_sync(0xffffffffu, dots[u], 2);
#pragma unroll
            for (int u = 0; u < 4; ++u) dots[u] += __shfl_xor_sync(0xffffffffu, dots[u], 4);
            if (sub == 0) {
#pragma unroll
                for (int u = 0; u < 4; ++u)
                    if (!decltype(guarded)::value || t0 + u < n) os[(t0 + u) * kScanBlockCols + warp * kScanCols + (lane >> 3)] = dots[u];
            }
        };
        for (int t0 = 0; t0 < n; t0 += 4) {
            if (t0 + 4 <= n) walk4(t0, std::false_type{});      // whole groups carry no per-token conditions
            else walk4(t0, std::true_type{});
        }
        __syncthreads();
        for (int i = threadIdx.x; i < n * kScanBlockCols; i += blockDim.x) {
            const int t = i / kScanBlockCols, c = block_col + i % kScanBlockCols;
            if (c < s.vdim) obuf[static_cast<size_t>(first + base + t) * o_ld + static_cast<size_t>(head) * s.vdim + c] = os[i];
        }
    }
    mlr_grid_dependents_may_start();     // only now: blocks of the next grid that wait on this SM slow the walk
    if (live) {
#pragma unroll
        for (int e = 0; e < E4; ++e)
#pragma unroll
            for (int j = 0; j < 4; ++j) my_state[static_cast<size_t>(my_col) * s.dim + 4 * (8 * e + sub) + j] = S[e][j];
    }
}


// Norm per head, weight, gate and the constant on the scan's float32 outputs [rows, heads * vdim].
template <typename T>
__global__ void __launch_bounds__(128) recurrence_readout_kernel(const float* obuf, const T* side, int ld_side, T* out, int ld_out,
                                                                 RecurrenceSpec s) {
    mlr_grid_wait();
    const int row = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    __shared__ float scratch[32];
    float inv_all = 1.0f;
    if (s.norm_all && s.eps >= 0.0f) {
        const int total = s.heads * s.vdim;
        const float* o = obuf + static_cast<size_t>(row) * total;
        float sum = 0.0f;
        for (int c = threadIdx.x; c < total; c += blockDim.x) {
            const float v = __ldcg(o + c);
            sum = fmaf(v, v, sum);
        }
        inv_all = 1.0f / sqrtf(mlr_block_sum(sum, scratch) / static_cast<float>(total) + s.eps);
    }
    for (int head = warp; head < s.heads; head += warps) {
        const float* o = obuf + (static_cast<size_t>(row) * s.heads + head) * s.vdim;
        float inv = inv_all;
        if (s.eps >= 0.0f && !s.norm_all) {
            float sum = 0.0f;
            for (int c = lane; c < s.vdim; c += 32) {
                const float v = __ldcg(o + c);
                sum = fmaf(v, v, sum);
            }
            inv = 1.0f / sqrtf(mlr_warp_sum(sum) / static_cast<float>(s.vdim) + s.eps);
        }
        const T* grow = side + static_cast<size_t>(row) * ld_side;
        T* orow = out + static_cast<size_t>(row) * ld_out + static_cast<size_t>(head) * s.vdim;
        for (int c = lane; c < s.vdim; c += 32) {
            float value = __ldcg(o + c) * inv;
            if (s.out_weight) value *= s.out_weight[s.norm_all ? head * s.vdim + c : c];
            if (s.gate_kind) {
                const float g = mlr_load(grow, s.col_gate + head * s.vdim + c);
                const float sig = 1.0f / (1.0f + expf(-g));
                value *= s.gate_kind == 2 ? g * sig : sig;
            }
            mlr_store(orow, c, value * s.out_scale);
        }
    }
    mlr_grid_dependents_may_start();
}

template <typename T>
__global__ void __launch_bounds__(256) short_conv_kernel(const T* in, int ld_in, T* out, int ld_out, int channels, int taps,
                                                         const float* weights, const float* state, long long state_stride,
                                                         const int* segment_info, const int* segment_of_row) {
    mlr_grid_wait();
    const int row = blockIdx.x;
    const int segment = segment_of_row[row];
    const int first = segment_info[4 * segment], slot = segment_info[4 * segment + 3];
    const int j = row - first;
    const float* old = state + static_cast<size_t>(slot) * state_stride;
    for (int c = threadIdx.x; c < channels; c += blockDim.x) {
        float y = 0.0f;
        for (int i = 0; i < taps; ++i) {
            const int m = j - (taps - 1) + i;      // the input this tap sees, counted from the step's first token
            const float x = m >= 0 ? mlr_load(in + static_cast<size_t>(first + m) * ld_in, c)
                                   : old[static_cast<size_t>(taps - 1 + m) * channels + c];
            y = fmaf(weights[static_cast<size_t>(c) * taps + i], x, y);
        }
        mlr_store(out + static_cast<size_t>(row) * ld_out, c, y / (1.0f + expf(-y)));
    }
    mlr_grid_dependents_may_start();
}

constexpr int kMaxTaps = 16;

template <typename T>
__global__ void __launch_bounds__(256) short_conv_state_kernel(const T* in, int ld_in, int channels, int taps, float* state,
                                                               long long state_stride, const int* segment_info) {
    mlr_grid_wait();
    const int segment = blockIdx.x;
    const int first = segment_info[4 * segment], count = segment_info[4 * segment + 1], slot = segment_info[4 * segment + 3];
    float* mine = state + static_cast<size_t>(slot) * state_stride;
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < channels; c += gridDim.y * blockDim.x) {
        float kept[kMaxTaps];
        for (int i = 0; i < taps - 1; ++i) kept[i] = mine[static_cast<size_t>(i) * channels + c];
        for (int i = 0; i < taps - 1; ++i) {
            const int m = count - (taps - 1) + i;
            mine[static_cast<size_t>(i) * channels + c] =
                m >= 0 ? mlr_load(in + static_cast<size_t>(first + m) * ld_in, c) : kept[taps - 1 + m];
        }
    }
    mlr_grid_dependents_may_start();
}

}  // namespace

MLR_API int mlr_linear_recurrence(const RecurrenceSpec* spec, const void* proj, int ld, const void* side, int ld_side, int act_bf16, void* out, int ld_out,
                                  float* state, long long state_stride, const int* segment_info, int n_segments, int rows, float* obuf,
                                  int* status, cudaStream_t stream) {
    // `obuf` (float32 [rows, heads * vdim], or null): the kernel leaves its plain outputs there and the read-out is a
    // launch of its own over the step's `rows` rows; a description with norm_all needs it.
    (void)status;
    MLR_REQUIRE(spec, "linear_recurrence: no description");
    const RecurrenceSpec& s = *spec;
    MLR_REQUIRE(s.heads > 0 && s.qk_heads > 0 && s.heads % s.qk_heads == 0 && s.heads <= 65535,
                "linear_recurrence: %d heads cannot share %d q/k heads", s.heads, s.qk_heads);
    MLR_REQUIRE(s.dim >= 1 && s.dim <= 256 && s.vdim >= 1 && s.vdim <= 256 && !(s.dim > 128 && s.vdim > 128),
                "linear_recurrence: a state of %d x %d per head is more than a block's registers hold (256 x 128 or 128 x 256)", s.dim, s.vdim);
    MLR_REQUIRE(s.prep != 1 || (s.rot_dims >= 0 && s.rot_dims % 2 == 0 && s.rot_dims <= s.dim && (s.rot_dims == 0 || s.freq)),
                "linear_recurrence: %d rotated values do not fit a head of %d", s.rot_dims, s.dim);
    MLR_REQUIRE(s.rule == 0 ? s.decay != nullptr : (s.rule == 1 && s.a_log && s.dt_bias), "linear_recurrence: the rule's constants are missing");
    MLR_REQUIRE(n_segments >= 0 && state && proj && side && out, "linear_recurrence: bad arguments");
    MLR_REQUIRE(!s.norm_all || obuf, "linear_recurrence: a norm over all heads needs the buffer of plain outputs");
    if (n_segments == 0) return 0;
    const int cols = s.vdim > 128 ? 8 : 4;
    const int warps = (s.vdim + cols - 1) / cols;
    const int regs = s.dim <= 32 ? 1 : s.dim <= 64 ? 2 : s.dim <= 128 ? 4 : 8;
    const size_t per_token = sizeof(float) * (2 * static_cast<size_t>(s.dim) + 2 * s.vdim + 2);
    int batch = static_cast<int>((40 * 1024) / per_token);
    batch = batch < 1 ? 1 : (batch > 32 ? 32 : batch);
    const size_t shared = per_token * batch;
    const dim3 grid(n_segments, s.heads);
#define MLR_GO(T, R, C)                                                                                                     \
    mlr_launch((linear_recurrence_kernel<T, R, C>), dim3(grid), dim3(warps * 32), shared, stream, static_cast<const T*>(proj), ld, static_cast<const T*>(side), ld_side, \
               static_cast<T*>(out), ld_out, state, state_stride, segment_info, s, batch, obuf)
#define MLR_PICK(T)                                              \
    do {                                                         \
        if (cols == 4) {                                         \
            if (regs == 1) MLR_GO(T, 1, 4);                      \
            else if (regs == 2) MLR_GO(T, 2, 4);                 \
            else if (regs == 4) MLR_GO(T, 4, 4);                 \
            else MLR_GO(T, 8, 4);                                \
        } else {                                                 \
            if (regs == 1) MLR_GO(T, 1, 8);                      \
            else if (regs == 2) MLR_GO(T, 2, 8);                 \
            else MLR_GO(T, 4, 8);                                \
        }                                                        \
    } while (0)
    if (act_bf16) MLR_PICK(__nv_bfloat16);
    else MLR_PICK(float);
#undef MLR_PICK
#undef MLR_GO
    if (obuf && rows > 0) {
        if (act_bf16)
            mlr_launch((recurrence_readout_kernel<__nv_bfloat16>), dim3(rows), dim3(128), 0, stream, obuf, static_cast<const __nv_bfloat16*>(side),
                       ld_side, static_cast<__nv_bfloat16*>(out), ld_out, s);
        else
            mlr_launch((recurrence_readout_kernel<float>), dim3(rows), dim3(128), 0, stream, obuf, static_cast<const float*>(side), ld_side,
                       static_cast<float*>(out), ld_out, s);
    }
    return mlr_launched("linear_recurrence");
}

static int check_recurrence(const RecurrenceSpec& s) {
    MLR_REQUIRE(s.heads > 0 && s.qk_heads > 0 && s.heads % s.qk_heads == 0 && s.heads <= 65535,
                "linear_recurrence: %d heads cannot share %d q/k heads", s.heads, s.qk_heads);
    MLR_REQUIRE(s.dim >= 1 && s.dim <= 256 && s.vdim >= 1 && s.vdim <= 256 && !(s.dim > 128 && s.vdim > 128),
                "linear_recurrence: a state of %d x %d per head is more than a block's registers hold (256 x 128 or 128 x 256)", s.dim, s.vdim);
    MLR_REQUIRE(s.prep != 1 || (s.rot_dims >= 0 && s.rot_dims % 2 == 0 && s.rot_dims <= s.dim && (s.rot_dims == 0 || s.freq)),
                "linear_recurrence: %d rotated values do not fit a head of %d", s.rot_dims, s.dim);
    MLR_REQUIRE(s.rule == 0 ? s.decay != nullptr : (s.rule == 1 && s.a_log && s.dt_bias), "linear_recurrence: the rule's constants are missing");
    return 0;
}

// The three-kernel form.  qf, kf: float32 [rows, qk_heads * dim]; gates: float32 [rows, 2 * heads] (delta rule; else unused);
// obuf: float32 [rows, heads * vdim].  Same results as `mlr_linear_recurrence` up to the order in which a column's sums are added
// (the same order for head sizes that are no multiple of 32).
MLR_API int mlr_linear_recurrence_split(const RecurrenceSpec* spec, const void* proj, int ld, const void* side, int ld_side, int act_bf16,
                                        void* out, int ld_out, float* state, long long state_stride, const int* segment_info,
                                        int n_segments, const int* positions, int rows, float* qf, float* kf, float* gates, float* obuf,
                                        cudaStream_t stream) {
    MLR_REQUIRE(spec, "linear_recurrence_split: no description");
    const RecurrenceSpec& s = *spec;
    if (check_recurrence(s)) return 1;
    MLR_REQUIRE(n_segments >= 0 && rows >= 0 && state && proj && side && out && qf && kf && obuf && positions && (s.rule == 0 || gates),
                "linear_recurrence_split: bad arguments");
    if (n_segments == 0 || rows == 0) return 0;
    const int regs = s.dim <= 32 ? 1 : s.dim <= 64 ? 2 : s.dim <= 128 ? 4 : 8;
    const size_t per_token = sizeof(float) * (4 * static_cast<size_t>(s.dim) + 2 * kScanBlockCols + 2);    // q and k in two stages
    int batch = static_cast<int>((44 * 1024) / per_token);
    batch = batch < 1 ? 1 : (batch > 32 ? 32 : batch);
    const size_t shared = per_token * batch;
    const dim3 grid(n_segments, s.heads, (s.vdim + kScanBlockCols - 1) / kScanBlockCols);
#define MLR_SCAN8(T, E)                                                                                                                \
    mlr_launch((recurrence_scan8_kernel<T, E>), dim3(grid), dim3(kScanWarps * 32), shared, stream, qf, kf, gates,                      \
               static_cast<const T*>(proj), ld, obuf, state, state_stride, segment_info, s, batch)
#define MLR_SPLIT(T)                                                                                                                   \
    do {                                                                                                                               \
        mlr_launch((recurrence_prepare_kernel<T>), dim3(rows), dim3(128), 0, stream, static_cast<const T*>(proj), ld,                  \
                   static_cast<const T*>(side), ld_side, qf, kf, gates, positions, s);                                                 \
        if (s.dim == 32) MLR_SCAN8(T, 1);                                                                                              \
        else if (s.dim == 64) MLR_SCAN8(T, 2);                                                                                         \
        else if (s.dim == 96) MLR_SCAN8(T, 3);                                                                                         \
        else if (s.dim == 128) MLR_SCAN8(T, 4);                                                                                        \
        else if (s.dim == 256) MLR_SCAN8(T, 8);                                                                                        \
        else if (regs == 1) mlr_launch((recurrence_scan_kernel<T, 1>), dim3(grid), dim3(kScanWarps * 32), shared, stream, qf, kf, gates,    \
                                  static_cast<const T*>(proj), ld, obuf, state, state_stride, segment_info, s, batch);                 \
        else if (regs == 2) mlr_launch((recurrence_scan_kernel<T, 2>), dim3(grid), dim3(kScanWarps * 32), shared, stream, qf, kf, gates, \
                                       static_cast<const T*>(proj), ld, obuf, state, state_stride, segment_info, s, batch);            \
        else if (regs == 4) mlr_launch((recurrence_scan_kernel<T, 4>), dim3(grid), dim3(kScanWarps * 32), shared, stream, qf, kf, gates, \
                                       static_cast<const T*>(proj), ld, obuf, state, state_stride, segment_info, s, batch);            \
        else mlr_launch((recurrence_scan_kernel<T, 8>), dim3(grid), dim3(kScanWarps * 32), shared, stream, qf, kf, gates,              \
                        static_cast<const T*>(proj), ld, obuf, state, state_stride, segment_info, s, batch);                           \
        mlr_launch((recurrence_readout_kernel<T>), dim3(rows), dim3(128), 0, stream, obuf, static_cast<const T*>(side), ld_side,       \
                   static_cast<T*>(out), ld_out, s);                                                                                   \
    } while (0)
    if (act_bf16) MLR_SPLIT(__nv_bfloat16);
    else MLR_SPLIT(float);
#undef MLR_SPLIT
#undef MLR_SCAN8
    return mlr_launched("linear_recurrence_split");
}

MLR_API int mlr_short_conv(const void* in, int ld_in, void* out, int ld_out, int act_bf16, int channels, int taps,
                           const float* weights, const float* state, long long state_stride, const int* segment_info,
                           const int* segment_of_row, int rows, cudaStream_t stream) {
    MLR_REQUIRE(channels > 0 && taps >= 1 && taps <= kMaxTaps, "short_conv: %d taps are outside [1, %d]", taps, kMaxTaps);
    MLR_REQUIRE(ld_in >= channels && ld_out >= channels && (taps == 1 || state), "short_conv: bad strides or no state");
    if (rows <= 0) return 0;
    if (act_bf16)
        mlr_launch((short_conv_kernel<__nv_bfloat16>), dim3(rows), dim3(256), 0, stream, static_cast<const __nv_bfloat16*>(in), ld_in,
                   static_cast<__nv_bfloat16*>(out), ld_out, channels, taps, weights, state, state_stride, segment_info, segment_of_row);
    else
        mlr_launch((short_conv_kernel<float>), dim3(rows), dim3(256), 0, stream, static_cast<const float*>(in), ld_in,
                   static_cast<float*>(out), ld_out, channels, taps, weights, state, state_stride, segment_info, segment_of_row);
    return mlr_launched("short_conv");
}

MLR_API int mlr_short_conv_state(const void* in, int ld_in, int act_bf16, int channels, int taps, float* state,
                                 long long state_stride, const int* segment_info, int n_segments, cudaStream_t stream) {
    MLR_REQUIRE(channels > 0 && taps >= 1 && taps <= kMaxTaps, "short_conv_state: %d taps are outside [1, %d]", taps, kMaxTaps);
    if (n_segments <= 0 || taps == 1) return 0;
    const dim3 grid(n_segments, (channels + 255) / 256);
    if (act_bf16)
        mlr_launch((short_conv_state_kernel<__nv_bfloat16>), dim3(grid), dim3(256), 0, stream, static_cast<const __nv_bfloat16*>(in), ld_in,
                   channels, taps, state, state_stride, segment_info);
    else
        mlr_launch((short_conv_state_kernel<float>), dim3(grid), dim3(256), 0, stream, static_cast<const float*>(in), ld_in, channels,
                   taps, state, state_stride, segment_info);
    return mlr_launched("short_conv_state");
}
