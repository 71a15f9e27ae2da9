// A routed feed-forward (mixture of experts) in five kernels, none of which needs the host to know how many
// tokens an expert received, so a step can be captured:
//
//   moe_route   : one block per token.  Router logits z = W_r h in 32-bit (ascending order of the sum),
//                 scores s = softmax(z) over all outputs, choice scores s + correction, restricted to the
//                 `keep` groups (of `count` equal groups of neighbours) whose best choice score is largest;
//                 the `top` largest choice scores win (ties: the lower index); the weights are their plain
//                 scores s.  The last `identity` outputs are experts without tensors whose output is the
//                 token itself: their weights are summed into id_weight[token].
//   moe_sort    : one block.  Counts the (token, choice) pairs of every real expert, lays the experts out one
//                 after the other (offsets) and gives every pair its place (slot_of_pair, pair_of_slot).
//   moe_up      : act[slot] = f(W_gate x, W_up x) for the pairs of each expert, a tile of TM pairs x 64
//                 columns per block; g = min(gate, limit), u = clamp(up, -limit, limit),
//                 f = g sigmoid(alpha g) (u + 1).
//   moe_down    : y[slot] = W_down act[slot], the same tiling, 32-bit output.
//   moe_combine : out[token] = T( sum_k weight_k y[slot(token, k)] + id_weight h[token] ).
//
// The products accumulate in 32-bit in ascending order of k whatever the tile a pair falls into, so a token's
// result does not depend on what else is in the step.
#include "common.cuh"

namespace {

constexpr int MAX_TOP = 32;
constexpr int MAX_OUTPUTS = 1024;

template <typename T>
__global__ void __launch_bounds__(128)
moe_route_kernel(const T* __restrict__ h, const T* __restrict__ w_router, const float* __restrict__ correction,
                 int* __restrict__ top_ids, float* __restrict__ top_w, float* __restrict__ id_weight, int hidden, int n_out,
                 int n_real, int top, int group_count, int group_keep) {
    __shared__ float z[MAX_OUTPUTS];
    __shared__ float choice[MAX_OUTPUTS];
    __shared__ float group_best[MAX_OUTPUTS];
    __shared__ unsigned char group_kept[MAX_OUTPUTS];
    pdl_launch_dependents();
    pdl_wait();
    const int64_t t = blockIdx.x;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const T* x = h + t * hidden;
    for (int e = warp; e < n_out; e += 4) {
        const T* w = w_router + (int64_t)e * hidden;
        float dot = 0.0f;
        for (int c = lane; c < hidden; c += 32) dot = fmaf(to_f32<T>(w[c]), to_f32<T>(x[c]), dot);
        dot = warp_sum(dot);
        if (lane == 0) z[e] = dot;
    }
    __syncthreads();
    if (tid != 0) return;
    float m = -INFINITY, sum = 0.0f;
    for (int e = 0; e < n_out; ++e) m = fmaxf(m, z[e]);
    for (int e = 0; e < n_out; ++e) {
        z[e] = expf(z[e] - m);
        sum += z[e];
    }
    const float inv = 1.0f / sum;
    for (int e = 0; e < n_out; ++e) {
        z[e] *= inv;
        choice[e] = z[e] + correction[e];
    }
    if (group_count > 1) {
        // a group's score is its best choice score; the `keep` best groups stay (of equal groups the earlier one)
        const int size = n_out / group_count;
        for (int g = 0; g < group_count; ++g) {
            float best = -INFINITY;
            for (int e = 0; e < size; ++e) best = fmaxf(best, choice[g * size + e]);
            group_best[g] = best;
            group_kept[g] = 0;
        }
        for (int k = 0; k < group_keep; ++k) {
            int best = -1;
            for (int g = 0; g < group_count; ++g)
                if (!group_kept[g] && (best < 0 || group_best[g] > group_best[best])) best = g;
            group_kept[best] = 1;
        }
        for (int e = 0; e < n_out; ++e)
            if (!group_kept[e / size]) choice[e] = -INFINITY;        // minus infinity, not 0: choice scores can be negative
    }
    float idw = 0.0f;
    for (int k = 0; k < top; ++k) {
        int best = -1;
        for (int e = 0; e < n_out; ++e)
            if (choice[e] > -INFINITY && (best < 0 || choice[e] > choice[best])) best = e;      // ties: the lower index
        if (best < 0) best = 0;                  // fewer candidates than `top` (the caller's sizes rule it out)
        choice[best] = -INFINITY;
        top_ids[t * top + k] = best;
        top_w[t * top + k] = z[best];
        if (best >= n_real) idw += z[best];
    }
    id_weight[t] = idw;
}

// counts [E + 1] (the last cell: pairs of identity experts), offsets [E + 1]
__global__ void __launch_bounds__(1024)
moe_sort_kernel(const int* __restrict__ top_ids, int n_pairs, int n_real, int* __restrict__ offsets, int* __restrict__ slot_of_pair,
                int* __restrict__ pair_of_slot) {
    extern __shared__ int counts[];            // [n_real] counts, then [n_real + 1] running offsets
    int* start = counts + n_real;
    pdl_launch_dependents();
    pdl_wait();
    for (int e = threadIdx.x; e < n_real; e += blockDim.x) counts[e] = 0;
    __syncthreads();
    for (int p = threadIdx.x; p < n_pairs; p += blockDim.x) {
        const int e = top_ids[p];
        if (e < n_real) atomicAdd(&counts[e], 1);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int run = 0;
        for (int e = 0; e < n_real; ++e) {
            start[e] = run;
            offsets[e] = run;
            run += counts[e];
        }
        start[n_real] = run;
        offsets[n_real] = run;
    }
    __syncthreads();
    for (int e = threadIdx.x; e < n_real; e += blockDim.x) counts[e] = 0;
    __syncthreads();
    for (int p = threadIdx.x; p < n_pairs; p += blockDim.x) {
        const int e = top_ids[p];
        int slot = -1;
        if (e < n_real) {
            slot = start[e] + atomicAdd(&counts[e], 1);
            pair_of_slot[slot] = p;
        }
        slot_of_pair[p] = slot;
    }
}

// Which expert and which of its row tiles block `tile` works on; false: beyond the last tile.
template <int TM>
__device__ __forceinline__ bool find_tile(const int* __restrict__ offsets, int n_real, int tile, int& expert, int& row0, int& rows) {
    int seen = 0;
    for (int e = 0; e < n_real; ++e) {
        const int n = offsets[e + 1] - offsets[e];
        const int tiles = (n + TM - 1) / TM;
        if (tile < seen + tiles) {
            expert = e;
            row0 = offsets[e] + (tile - seen) * TM;
            rows = min(TM, offsets[e + 1] - row0);
            return true;
        }
        seen += tiles;
    }
    return false;
}

constexpr int TN = 64, TK = 32;

// A tile of TM rows of X (gathered through `src_row`) times TN rows of W, accumulated over K in 32-bit on fmaf.
// 256 threads: thread (tx, ty) owns rows ty, ty + 16, ... (TM / 16 of them, at least 1 with TM = 8: ty < 8) and
// columns tx * 4 .. + 3.  DUAL: two weight matrices at once (gate and up).
template <typename T, int TM, bool DUAL>
__device__ __forceinline__ void tile_product(const T* __restrict__ X, int64_t x_stride, const int* src_row, int rows,
                                             const T* __restrict__ W0, const T* __restrict__ W1, int n_cols, int col0, int K,
                                             float (&acc0)[(TM + 15) / 16][4], float (&acc1)[(TM + 15) / 16][4], float* xs, float* ws0,
                                             float* ws1) {
    constexpr int RPT = (TM + 15) / 16;
    const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
#pragma unroll
    for (int a = 0; a < RPT; ++a)
#pragma unroll
        for (int b = 0; b < 4; ++b) acc0[a][b] = acc1[a][b] = 0.0f;
    for (int k0 = 0; k0 < K; k0 += TK) {
        __syncthreads();
        for (int x = tid; x < TM * TK; x += 256) {
            const int rr = x / TK, kk = x % TK;
            xs[rr * (TK + 1) + kk] = (rr < rows && k0 + kk < K) ? to_f32<T>(X[(int64_t)src_row[rr] * x_stride + k0 + kk]) : 0.0f;
        }
        for (int x = tid; x < TN * TK; x += 256) {
            const int cc = x / TK, kk = x % TK;
            const bool ok = col0 + cc < n_cols && k0 + kk < K;
            ws0[cc * (TK + 1) + kk] = ok ? to_f32<T>(W0[(int64_t)(col0 + cc) * K + k0 + kk]) : 0.0f;
            if (DUAL) ws1[cc * (TK + 1) + kk] = ok ? to_f32<T>(W1[(int64_t)(col0 + cc) * K + k0 + kk]) : 0.0f;
        }
        __syncthreads();
#pragma unroll 8
        for (int kk = 0; kk < TK; ++kk) {
            float wv0[4], wv1[4];
#pragma unroll
            for (int b = 0; b < 4; ++b) {
                wv0[b] = ws0[(tx * 4 + b) * (TK + 1) + kk];
                if (DUAL) wv1[b] = ws1[(tx * 4 + b) * (TK + 1) + kk];
            }
#pragma unroll
            for (int a = 0; a < RPT; ++a) {
                const int rr = ty + a * 16;
                if (rr < TM) {
                    const float xv = xs[rr * (TK + 1) + kk];
#pragma unroll
                    for (int b = 0; b < 4; ++b) {
                        acc0[a][b] = fmaf(xv, wv0[b], acc0[a][b]);
                        if (DUAL) acc1[a][b] = fmaf(xv, wv1[b], acc1[a][b]);
                    }
                }
            }
        }
    }
}

template <typename T, int TM>
__global__ void __launch_bounds__(256)
moe_up_kernel(const T* __restrict__ h, const T* __restrict__ w_gate_up, const int* __restrict__ offsets,
              const int* __restrict__ pair_of_slot, T* __restrict__ act, int n_real, int top, int hidden, int ff, float limit,
              float alpha) {
    __shared__ float xs[TM * (TK + 1)], ws0[TN * (TK + 1)], ws1[TN * (TK + 1)];
    __shared__ int src_row[TM];
    pdl_launch_dependents();
    pdl_wait();
    int expert, row0, rows;
    if (!find_tile<TM>(offsets, n_real, blockIdx.y, expert, row0, rows)) return;
    if (threadIdx.x < TM) src_row[threadIdx.x] = threadIdx.x < rows ? pair_of_slot[row0 + threadIdx.x] / top : 0;
    const int col0 = blockIdx.x * TN;
    const T* wg = w_gate_up + (int64_t)expert * 2 * ff * hidden;      // [gate rows; up rows] of the expert
    float g[(TM + 15) / 16][4], u[(TM + 15) / 16][4];
    tile_product<T, TM, true>(h, hidden, src_row, rows, wg, wg + (int64_t)ff * hidden, ff, col0, hidden, g, u, xs, ws0, ws1);
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
#pragma unroll
    for (int a = 0; a < (TM + 15) / 16; ++a) {
        const int rr = ty + a * 16;
        if (rr >= rows || rr >= TM) continue;
#pragma unroll
        for (int b = 0; b < 4; ++b) {
            const int c = col0 + tx * 4 + b;
            if (c >= ff) continue;
            const float gv = fminf(g[a][b], limit), uv = fminf(fmaxf(u[a][b], -limit), limit);
            act[(int64_t)(row0 + rr) * ff + c] = from_f32<T>(gv / (1.0f + expf(-alpha * gv)) * (uv + 1.0f));
        }
    }
}

template <typename T, int TM>
__global__ void __launch_bounds__(256)
moe_down_kernel(const T* __restrict__ act, const T* __restrict__ w_down, const int* __restrict__ offsets, float* __restrict__ y,
                int n_real, int hidden, int ff) {
    __shared__ float xs[TM * (TK + 1)], ws0[TN * (TK + 1)];
    __shared__ int src_row[TM];
    pdl_launch_dependents();
    pdl_wait();
    int expert, row0, rows;
    if (!find_tile<TM>(offsets, n_real, blockIdx.y, expert, row0, rows)) return;
    if (threadIdx.x < TM) src_row[threadIdx.x] = row0 + min((int)threadIdx.x, rows - 1);
    const int col0 = blockIdx.x * TN;
    float acc[(TM + 15) / 16][4], unused[(TM + 15) / 16][4];
    tile_product<T, TM, false>(act, ff, src_row, rows, w_down + (int64_t)expert * hidden * ff, nullptr, hidden, col0, ff, acc, unused,
                               xs, ws0, nullptr);
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
#pragma unroll
    for (int a = 0; a < (TM + 15) / 16; ++a) {
        const int rr = ty + a * 16;
        if (rr >= rows || rr >= TM) continue;
#pragma unroll
        for (int b = 0; b < 4; ++b) {
            const int c = col0 + tx * 4 + b;
            if (c < hidden) y[(int64_t)(row0 + rr) * hidden + c] = acc[a][b];
        }
    }
}

template <typename T>
__global__ void moe_combine_kernel(const float* __restrict__ y, const T* __restrict__ h, const int* __restrict__ slot_of_pair,
                                   const float* __restrict__ top_w, const float* __restrict__ id_weight, T* __restrict__ out,
                                   int top, int hidden) {
    pdl_launch_dependents();
    pdl_wait();
    const int64_t t = blockIdx.x;
    const float idw = id_weight[t];
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
        float v = idw != 0.0f ? idw * to_f32<T>(h[t * hidden + c]) : 0.0f;
        for (int k = 0; k < top; ++k) {
            const int slot = slot_of_pair[t * top + k];
            if (slot >= 0) v = fmaf(top_w[t * top + k], y[(int64_t)slot * hidden + c], v);
        }
        out[t * hidden + c] = from_f32<T>(v);
    }
}

template <typename T, int TM>
int moe_experts_launch(const T* h, const T* w_gate_up, const T* w_down, const int* offsets, const int* pair_of_slot, T* act, float* y,
                       int n_pairs, int n_real, int top, int hidden, int ff, float limit, float alpha, cudaStream_t stream) {
    const int tiles = (n_pairs + TM - 1) / TM + n_real;         // an upper bound on the row tiles of all experts together
    if (tiles > 65535) return Q3_ERR_TOO_LARGE;
    int code = (int)q3_launch(moe_up_kernel<T, TM>, dim3((ff + TN - 1) / TN, tiles), dim3(256), 0, stream, h, w_gate_up, offsets,
                              pair_of_slot, act, n_real, top, hidden, ff, limit, alpha);
    if (code != 0) return code;
    return (int)q3_launch(moe_down_kernel<T, TM>, dim3((hidden + TN - 1) / TN, tiles), dim3(256), 0, stream, act, w_down, offsets, y,
                          n_real, hidden, ff);
}

}  // namespace

#define Q3_MOE_EXPORTS(SUFFIX, T)                                                                                         \
    Q3_EXPORT int q3_moe_route_##SUFFIX(const void* h, const void* w_router, const float* correction, int* top_ids,       \
                                        float* top_w, float* id_weight, int64_t n_tokens, int hidden, int n_out, int n_real, \
                                        int top, int group_count, int group_keep, void* stream) {                         \
        if (n_tokens <= 0) return 0;                                                                                      \
        if (n_out <= 0 || n_out > MAX_OUTPUTS || top <= 0 || top > MAX_TOP || top > n_out || n_real < 0 || n_real > n_out || \
            group_count <= 0 || n_out % group_count != 0 || group_keep <= 0 || group_keep > group_count ||                \
            n_tokens > 0x7fffffffLL)                                                                                      \
            return Q3_ERR_BAD_SIZE;                                                                                       \
        return (int)q3_launch(moe_route_kernel<T>, dim3((unsigned)n_tokens), dim3(128), 0, (cudaStream_t)stream,          \
                              (const T*)h, (const T*)w_router, correction, top_ids, top_w, id_weight, hidden, n_out,      \
                              n_real, top, group_count, group_keep);                                                      \
    }                                                                                                                     \
    Q3_EXPORT int q3_moe_experts_##SUFFIX(const void* h, const void* w_gate_up, const void* w_down, const int* offsets,   \
                                          const int* pair_of_slot, void* act, float* y, int n_pairs, int n_real, int top, \
                                          int hidden, int ff, float limit, float alpha, void* stream) {                   \
        if (n_pairs <= 0 || n_real <= 0) return 0;                                                                        \
        if (n_pairs <= 64)                                                                                                \
            return moe_experts_launch<T, 8>((const T*)h, (const T*)w_gate_up, (const T*)w_down, offsets, pair_of_slot,    \
                                            (T*)act, y, n_pairs, n_real, top, hidden, ff, limit, alpha,                   \
                                            (cudaStream_t)stream);                                                        \
        return moe_experts_launch<T, 32>((const T*)h, (const T*)w_gate_up, (const T*)w_down, offsets, pair_of_slot,       \
                                         (T*)act, y, n_pairs, n_real, top, hidden, ff, limit, alpha, (cudaStream_t)stream); \
    }                                                                                                                     \
    Q3_EXPORT int q3_moe_combine_##SUFFIX(const float* y, const void* h, const int* slot_of_pair, const float* top_w,     \
                                          const float* id_weight, void* out, int64_t n_tokens, int top, int hidden,       \
                                          void* stream) {                                                                 \
        if (n_tokens <= 0) return 0;                                                                                      \
        if (n_tokens > 0x7fffffffLL) return Q3_ERR_BAD_SIZE;                                                              \
        return (int)q3_launch(moe_combine_kernel<T>, dim3((unsigned)n_tokens), dim3(hidden >= 1024 ? 256 : 128), 0,       \
                              (cudaStream_t)stream, y, (const T*)h, slot_of_pair, top_w, id_weight, (T*)out, top, hidden); \
    }

Q3_EXPORT int q3_moe_sort(const int* top_ids, int n_pairs, int n_real, int* offsets, int* slot_of_pair, int* pair_of_slot,
                          void* stream) {
    if (n_pairs <= 0) return 0;
    if (n_real < 0 || n_real > 4096) return Q3_ERR_BAD_SIZE;
    return (int)q3_launch(moe_sort_kernel, dim3(1), dim3(1024), (size_t)(2 * n_real + 1) * sizeof(int), (cudaStream_t)stream, top_ids,
                          n_pairs, n_real, offsets, slot_of_pair, pair_of_slot);
}

Q3_MOE_EXPORTS(f32, float)
Q3_MOE_EXPORTS(bf16, bf16)
