// Linear attention with a per-head decay ("lightning" attention) and a fixed-size state per sequence:
//
//     S_t = decay_h S_(t-1) + k_t v_t^T          (S: [d, vd] per head, float32, one per cache slot)
//     o_t = S_t^T q_t
//
// with q, k, v = SiLU of the projection output.  A row of the projection holds, head by head, the H*d
// values of q, the H*d of k, the H*vd of v and the H*vd of the output gate g.
//
//   lightning_scan  : one block per (head, sequence, tile of up to 64 columns of the state: columns do not
//                     depend on one another) walks the sequence's new tokens in order with its share of the
//                     state in registers: thread (j, r) owns column j of the tile and the rows r, r + R,
//                     r + 2R, ...; it reads the state from the slot's row before the first token and
//                     writes it back after the last.  A decode step is the same kernel with one token.
//                     The activation, the decay, the state and o are 32-bit whatever T.
//   lightning_chunks: the same recurrence for prompts, C = 32 tokens at a time:
//                     o_i = decay^(i+1) S_0^T q_i + sum_(j<=i) decay^(i-j) (q_i . k_j) v_j  and
//                     S_C = decay^C S_0 + sum_j decay^(C-1-j) k_j v_j^T, all in 32-bit; the powers are
//                     formed as exp2(n log2 decay), never as quotients, so a small decay cannot overflow.
//   gated_norm      : out = T( o / sqrt(mean(o^2) + eps) * w * sigmoid(g) ) over a token's H*vd values.
#include "common.cuh"

namespace {

__device__ __forceinline__ float silu_f32(float z) { return z / (1.0f + expf(-z)); }

constexpr int COL_TILE = 64;      // columns of the state per block
constexpr int MAX_THREADS = 512;

template <typename T, int ROWS>
__global__ void __launch_bounds__(MAX_THREADS) lightning_scan_kernel(const T* __restrict__ proj, float* __restrict__ state, const float* __restrict__ decay,
                                      const int* __restrict__ seq_start, const int* __restrict__ seq_slots,
                                      float* __restrict__ out, int H, int d, int vd, int R, int vt) {
    extern __shared__ float smem[];
    float* q_s = smem;                 // [d]
    float* k_s = q_s + d;              // [d]
    float* v_s = k_s + d;              // [vt]
    float* red = v_s + vt;             // [R][vt]
    pdl_launch_dependents();
    pdl_wait();
    const int head = blockIdx.x, seq = blockIdx.y, col0 = blockIdx.z * vt;
    const int tid = threadIdx.x, jt = tid % vt, j = col0 + jt, r = tid / vt;
    const bool live = r < R && j < vd;
    const float lam = decay[head];
    const int64_t cols = 2 * (int64_t)H * d + 2 * (int64_t)H * vd;
    float* S_g = state + ((int64_t)seq_slots[seq] * H + head) * d * vd;
    float S[ROWS];
#pragma unroll
    for (int n = 0; n < ROWS; ++n) {
        const int i = r + n * R;
        S[n] = live && i < d ? S_g[(int64_t)i * vd + j] : 0.0f;
    }
    for (int t = seq_start[seq]; t < seq_start[seq + 1]; ++t) {
        const T* row = proj + t * cols;
        for (int i = tid; i < d; i += blockDim.x) {
            q_s[i] = silu_f32(to_f32<T>(row[(int64_t)head * d + i]));
            k_s[i] = silu_f32(to_f32<T>(row[(int64_t)(H + head) * d + i]));
        }
        for (int i = tid; i < vt; i += blockDim.x)
            v_s[i] = col0 + i < vd ? silu_f32(to_f32<T>(row[2 * (int64_t)H * d + (int64_t)head * vd + col0 + i])) : 0.0f;
        __syncthreads();
        if (live) {
            const float v = v_s[jt];
            float part = 0.0f;
#pragma unroll
            for (int n = 0; n < ROWS; ++n) {
                const int i = r + n * R;
                if (i < d) {
                    S[n] = fmaf(lam, S[n], k_s[i] * v);
                    part = fmaf(S[n], q_s[i], part);
                }
            }
            red[r * vt + jt] = part;
        }
        __syncthreads();
        if (tid < vt && col0 + tid < vd) {
            float o = 0.0f;
            for (int rr = 0; rr < R; ++rr) o += red[rr * vt + tid];
            out[((int64_t)t * H + head) * vd + col0 + tid] = o;
        }
    }
    if (live) {
#pragma unroll
        for (int n = 0; n < ROWS; ++n) {
            const int i = r + n * R;
            if (i < d) S_g[(int64_t)i * vd + j] = S[n];
        }
    }
}

template <typename T>
int lightning_scan_launch(const T* proj, float* state, const float* decay, const int* seq_start, const int* seq_slots, float* out,
                          int n_seqs, int H, int d, int vd, cudaStream_t stream) {
    if (n_seqs <= 0) return 0;
    if (H <= 0 || d <= 0 || vd <= 0 || d > 256 || vd > 256 || n_seqs > 65535) return Q3_ERR_BAD_SIZE;
    const int vt = min(vd, COL_TILE);
    const int R = min(d, MAX_THREADS / vt);            // row slices: as many as a block holds
    const int rows = (d + R - 1) / R;                  // at most 32: d <= 256, R >= 8 unless d is smaller
    const int threads = ((vt * R + 31) / 32) * 32;
    const size_t smem = (size_t)(2 * d + vt + R * vt) * sizeof(float);
    const dim3 grid(H, n_seqs, (vd + vt - 1) / vt);
#define Q3_SCAN(ROWS)                                                                                                    \
    return (int)q3_launch(lightning_scan_kernel<T, ROWS>, grid, dim3(threads), smem, stream, proj, state, decay, seq_start, \
                          seq_slots, out, H, d, vd, R, vt)
    if (rows <= 1) Q3_SCAN(1);
    if (rows <= 2) Q3_SCAN(2);
    if (rows <= 4) Q3_SCAN(4);
    if (rows <= 8) Q3_SCAN(8);
    if (rows <= 16) Q3_SCAN(16);
    Q3_SCAN(32);
#undef Q3_SCAN
}

// ---------------------------------------------------------------- prompts, a chunk of tokens at a time
// One block per (head, sequence, tile of columns), as in the scan.  Per chunk of C tokens the block holds q, k
// (C x d), its columns of v and the C x C matrix of decayed scores in shared memory and its share of the state in
// registers: thread (j, r) owns column j and rows r, r + R, ...  All sums run in ascending order of their index.
constexpr int CHUNK = 32;

template <typename T, int ROWS>
__global__ void __launch_bounds__(MAX_THREADS) lightning_chunks_kernel(const T* __restrict__ proj, float* __restrict__ state, const float* __restrict__ decay,
                                        const int* __restrict__ seq_start, const int* __restrict__ seq_slots,
                                        float* __restrict__ out, int H, int d, int vd, int R, int vt) {
    extern __shared__ float smem[];
    float* q_s = smem;                         // [C][d + 1]
    float* k_s = q_s + CHUNK * (d + 1);        // [C][d + 1]
    float* v_s = k_s + CHUNK * (d + 1);        // [C][vt]
    float* a_s = v_s + CHUNK * vt;             // [C][C + 1]: decay^(i-j) (q_i . k_j), j <= i
    float* red = a_s + CHUNK * (CHUNK + 1);    // [R][C][vt] partial S_0^T q_i
    __shared__ float pw[CHUNK + 1];            // decay^n
    pdl_launch_dependents();
    pdl_wait();
    const int head = blockIdx.x, seq = blockIdx.y, col0 = blockIdx.z * vt;
    const int tid = threadIdx.x, nthreads = blockDim.x, jt = tid % vt, j = col0 + jt, r = tid / vt;
    const bool live = r < R && j < vd;
    const float lam = decay[head];
    const float l2 = lam > 0.0f ? log2f(lam) : 0.0f;
    for (int n = tid; n <= CHUNK; n += nthreads) pw[n] = n == 0 ? 1.0f : (lam > 0.0f ? exp2f((float)n * l2) : 0.0f);
    const int64_t cols = 2 * (int64_t)H * d + 2 * (int64_t)H * vd;
    const int dp = d + 1;
    float* S_g = state + ((int64_t)seq_slots[seq] * H + head) * d * vd;
    float S[ROWS];
#pragma unroll
    for (int n = 0; n < ROWS; ++n) {
        const int i = r + n * R;
        S[n] = live && i < d ? S_g[(int64_t)i * vd + j] : 0.0f;
    }
    const int t_end = seq_start[seq + 1];
    for (int t0 = seq_start[seq]; t0 < t_end; t0 += CHUNK) {
        const int C = min(CHUNK, t_end - t0);
        __syncthreads();                                   // the chunk before is done with the buffers
        for (int x = tid; x < C * d; x += nthreads) {
            const int i = x / d, c = x % d;
            const T* row = proj + (int64_t)(t0 + i) * cols;
            q_s[i * dp + c] = silu_f32(to_f32<T>(row[(int64_t)head * d + c]));
            k_s[i * dp + c] = silu_f32(to_f32<T>(row[(int64_t)(H + head) * d + c]));
        }
        for (int x = tid; x < C * vt; x += nthreads) {
            const int i = x / vt, c = col0 + x % vt;
            v_s[x] = c < vd ? silu_f32(to_f32<T>(proj[(int64_t)(t0 + i) * cols + 2 * (int64_t)H * d + (int64_t)head * vd + c])) : 0.0f;
        }
        __syncthreads();
        // scores inside the chunk
        for (int x = tid; x < C * C; x += nthreads) {
            const int i = x / C, jj = x % C;
            float dot = 0.0f;
            if (jj <= i) {
                for (int c = 0; c < d; ++c) dot = fmaf(q_s[i * dp + c], k_s[jj * dp + c], dot);
                dot *= pw[i - jj];
            }
            a_s[i * (CHUNK + 1) + jj] = dot;
        }
        // what the state before the chunk gives every token: partial sums over this thread's rows
        if (live) {
            for (int i = 0; i < C; ++i) {
                float part = 0.0f;
#pragma unroll
                for (int n = 0; n < ROWS; ++n) {
                    const int row = r + n * R;
                    if (row < d) part = fmaf(S[n], q_s[i * dp + row], part);
                }
                red[(r * CHUNK + i) * vt + jt] = part;
            }
        }
        __syncthreads();
        // o_i = decay^(i+1) * (S_0^T q_i) + sum_j a_ij v_j
        for (int x = tid; x < C * vt; x += nthreads) {
            const int i = x / vt, c = x % vt;
            if (col0 + c >= vd) continue;
            float inter = 0.0f;
            for (int rr = 0; rr < R; ++rr) inter += red[(rr * CHUNK + i) * vt + c];
            float intra = 0.0f;
            for (int jj = 0; jj <= i; ++jj) intra = fmaf(a_s[i * (CHUNK + 1) + jj], v_s[jj * vt + c], intra);
            out[((int64_t)(t0 + i) * H + head) * vd + col0 + c] = fmaf(pw[i + 1], inter, intra);
        }
        // the state after the chunk
        if (live) {
#pragma unroll
            for (int n = 0; n < ROWS; ++n) {
                const int row = r + n * R;
                if (row < d) {
                    float add = 0.0f;
                    for (int jj = 0; jj < C; ++jj) add = fmaf(pw[C - 1 - jj] * k_s[jj * dp + row], v_s[jj * vt + jt], add);
                    S[n] = fmaf(pw[C], S[n], add);
                }
            }
        }
    }
    if (live) {
#pragma unroll
        for (int n = 0; n < ROWS; ++n) {
            const int i = r + n * R;
            if (i < d) S_g[(int64_t)i * vd + j] = S[n];
        }
    }
}

template <typename T>
int lightning_chunks_launch(const T* proj, float* state, const float* decay, const int* seq_start, const int* seq_slots,
                            float* out, int n_seqs, int H, int d, int vd, cudaStream_t stream) {
    if (n_seqs <= 0) return 0;
    if (H <= 0 || d <= 0 || vd <= 0 || d > 256 || vd > 256 || n_seqs > 65535) return Q3_ERR_BAD_SIZE;
    // narrower column tiles while the blocks are fewer than the multiprocessors: a prompt of one sequence has only
    // heads x tiles blocks, and a block's work per chunk shrinks with its tile (the scores alone are computed by every tile)
    int vt = min(vd, COL_TILE);
    while (vt > 16 && (int64_t)H * n_seqs * ((vd + vt - 1) / vt) < q3_device_sm_count()) vt /= 2;
    const int R = min(d, MAX_THREADS / vt);
    const int rows = (d + R - 1) / R;
    const int threads = ((vt * R + 31) / 32) * 32;
    const size_t smem = (size_t)(2 * CHUNK * (d + 1) + CHUNK * vt + CHUNK * (CHUNK + 1) + R * CHUNK * vt) * sizeof(float);
    if (smem > 200 * 1024) return Q3_ERR_BAD_SIZE;
    const dim3 grid(H, n_seqs, (vd + vt - 1) / vt);
    static Q3PerDevice allowed[6];
#define Q3_CHUNKS(ROWS, SLOT)                                                                                             \
    {                                                                                                                     \
        if (smem > 48 * 1024) {                                                                                           \
            const cudaError_t e = q3_allow_shared_memory(lightning_chunks_kernel<T, ROWS>, 200 * 1024, allowed[SLOT]);     \
            if (e != cudaSuccess) return (int)e;                                                                          \
        }                                                                                                                 \
        return (int)q3_launch(lightning_chunks_kernel<T, ROWS>, grid, dim3(threads), smem, stream, proj, state, decay,     \
                              seq_start, seq_slots, out, H, d, vd, R, vt);                                                \
    }
    if (rows <= 1) Q3_CHUNKS(1, 0)
    if (rows <= 2) Q3_CHUNKS(2, 1)
    if (rows <= 4) Q3_CHUNKS(4, 2)
    if (rows <= 8) Q3_CHUNKS(8, 3)
    if (rows <= 16) Q3_CHUNKS(16, 4)
    Q3_CHUNKS(32, 5)
#undef Q3_CHUNKS
}

// ---------------------------------------------------------------- unit rms over all heads, weight, sigmoid gate
template <typename T>
__global__ void gated_norm_kernel(const float* __restrict__ o, const T* __restrict__ gate, int64_t gate_stride,
                                  const float* __restrict__ w, float eps, T* __restrict__ out, int size) {
    __shared__ float scratch[33];
    pdl_launch_dependents();
    pdl_wait();
    const int64_t t = blockIdx.x;
    const float* row = o + t * size;
    float sq = 0.0f;
    for (int c = threadIdx.x; c < size; c += blockDim.x) sq += row[c] * row[c];
    const float inv = rsqrtf(block_sum(sq, scratch) / (float)size + eps);
    for (int c = threadIdx.x; c < size; c += blockDim.x) {
        const float g = to_f32<T>(gate[t * gate_stride + c]);
        out[t * size + c] = from_f32<T>(row[c] * inv * w[c] / (1.0f + expf(-g)));
    }
}

}  // namespace

#define Q3_LIGHTNING_EXPORTS(SUFFIX, T)                                                                                   \
    Q3_EXPORT int q3_lightning_scan_##SUFFIX(const void* proj, float* state, const float* decay, const int* seq_start,    \
                                             const int* seq_slots, float* out, int n_seqs, int heads, int d, int vd,      \
                                             void* stream) {                                                              \
        return lightning_scan_launch<T>((const T*)proj, state, decay, seq_start, seq_slots, out, n_seqs, heads, d, vd,    \
                                        (cudaStream_t)stream);                                                            \
    }                                                                                                                     \
    Q3_EXPORT int q3_lightning_chunks_##SUFFIX(const void* proj, float* state, const float* decay, const int* seq_start,  \
                                               const int* seq_slots, float* out, int n_seqs, int heads, int d, int vd,    \
                                               void* stream) {                                                            \
        return lightning_chunks_launch<T>((const T*)proj, state, decay, seq_start, seq_slots, out, n_seqs, heads, d, vd,  \
                                          (cudaStream_t)stream);                                                          \
    }                                                                                                                     \
    Q3_EXPORT int q3_gated_norm_##SUFFIX(const float* o, const void* gate, int64_t gate_stride, const float* w, float eps, \
                                         void* out, int64_t n_tokens, int size, void* stream) {                           \
        if (n_tokens <= 0) return 0;                                                                                      \
        if (size <= 0 || n_tokens > 0x7fffffffLL) return Q3_ERR_BAD_SIZE;                                                 \
        return (int)q3_launch(gated_norm_kernel<T>, dim3((unsigned)n_tokens), dim3(size >= 1024 ? 256 : 128), 0,          \
                              (cudaStream_t)stream, o, (const T*)gate, gate_stride, w, eps, (T*)out, size);               \
    }

Q3_LIGHTNING_EXPORTS(f32, float)
Q3_LIGHTNING_EXPORTS(bf16, bf16)
