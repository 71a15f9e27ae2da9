// Kernels for a hidden state that travels as S streams per token (hyper-connections), kept in
// 32-bit whatever the compute type T of the matrix products.  Layout: streams [token, S, hidden].
//
//   embedding_streams : streams[t][s] = table[ids[t]] * scale for every s                  (T -> float)
//   hyper_norm        : ONE pass over a token's streams that
//                         (1) settles the sublayer output y that is still pending,
//                               x_to <- sum_from mix[from][to] x_from + out[to] y      (all streams at once),
//                         (2) forms the next sublayer's input u = sum_s in[s] x_s,
//                         (3) normalises it, r = u / sqrt(mean(u^2) + eps) * w, and rounds r to T.
//                       Any of the three may be left out: no pending output (the first sublayer), no
//                       result (settle only), no normalisation (u itself is written).  With `rows` the
//                       kernel works on the listed tokens only and leaves the streams as they are: the
//                       model's tail, where only the wanted rows are summed and normalised.
//
// S = 1 with mix = [1] and in = [1] is the plain residual sum x <- x + out y.  Coefficients, sums
// and statistics are 32-bit; only the result is rounded.
#include "common.cuh"

namespace {

constexpr int MAX_STREAMS = 16;

template <typename T>
__global__ void embedding_streams_kernel(const int* __restrict__ ids, const T* __restrict__ table, float* __restrict__ out,
                                         int hidden, int vocab, float scale, int copies) {
    pdl_launch_dependents();
    pdl_wait();
    const int64_t t = blockIdx.x;
    const int id = ids[t];
    const bool ok = id >= 0 && id < vocab;                 // an id outside the table gives zero rows
    const T* src = table + (int64_t)(ok ? id : 0) * hidden;
    float* dst = out + t * copies * hidden;
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
        const float v = ok ? to_f32<T>(src[c]) * scale : 0.0f;
        for (int s = 0; s < copies; ++s) dst[(int64_t)s * hidden + c] = v;
    }
}

// One block per row of the result.  The sum u of a token is kept in shared memory between the two passes.  VEC = 4:
// 16-byte accesses to the streams (a hidden size in steps of 4); VEC = 1: any size.  SMAX bounds the streams a thread
// keeps in registers (4 with 16-byte accesses, MAX_STREAMS without).
template <typename T, typename TO, int VEC, int SMAX>
__global__ void __launch_bounds__(512) hyper_norm_kernel(float* __restrict__ streams, const T* __restrict__ branch, const float* __restrict__ mix,
                                  const float* __restrict__ out_coef, const float* __restrict__ in_coef,
                                  const float* __restrict__ norm_w, float eps, TO* __restrict__ out,
                                  const int* __restrict__ rows, int S, int hidden, int normalize) {
    extern __shared__ float u_s[];
    __shared__ float scratch[33];
    __shared__ float c_mix[MAX_STREAMS * MAX_STREAMS], c_out[MAX_STREAMS], c_in[MAX_STREAMS];
    pdl_launch_dependents();
    pdl_wait();
    const int64_t r = blockIdx.x;
    const int64_t t = rows != nullptr ? rows[r] : r;
    const bool write_streams = rows == nullptr && branch != nullptr;
    for (int i = threadIdx.x; i < S * S && branch != nullptr; i += blockDim.x) c_mix[i] = mix[i];
    for (int i = threadIdx.x; i < S; i += blockDim.x) {
        c_out[i] = branch != nullptr ? out_coef[i] : 0.0f;
        c_in[i] = in_coef != nullptr ? in_coef[i] : 1.0f;
    }
    __syncthreads();
    float* xs = streams + t * S * hidden;
    const T* y = branch != nullptr ? branch + t * hidden : nullptr;
    float sq = 0.0f;
    for (int c = threadIdx.x * VEC; c < hidden; c += blockDim.x * VEC) {
        float x[SMAX][VEC], yv[VEC], u[VEC];
#pragma unroll
        for (int s = 0; s < SMAX; ++s) {
            if (s < S) {
                if constexpr (VEC == 4) {
                    const float4 v = *reinterpret_cast<const float4*>(xs + (int64_t)s * hidden + c);
                    x[s][0] = v.x; x[s][1] = v.y; x[s][2] = v.z; x[s][3] = v.w;
                } else {
                    x[s][0] = xs[(int64_t)s * hidden + c];
                }
            }
        }
#pragma unroll
        for (int i = 0; i < VEC; ++i) u[i] = 0.0f;
        if (y != nullptr) {
#pragma unroll
            for (int i = 0; i < VEC; ++i) yv[i] = to_f32<T>(y[c + i]);
#pragma unroll
            for (int to = 0; to < SMAX; ++to) {
                if (to < S) {
                    float v[VEC];
#pragma unroll
                    for (int i = 0; i < VEC; ++i) v[i] = 0.0f;
#pragma unroll
                    for (int from = 0; from < SMAX; ++from)
                        if (from < S) {
#pragma unroll
                            for (int i = 0; i < VEC; ++i) v[i] = fmaf(c_mix[from * S + to], x[from][i], v[i]);
                        }
#pragma unroll
                    for (int i = 0; i < VEC; ++i) {
                        v[i] = fmaf(c_out[to], yv[i], v[i]);
                        u[i] = fmaf(c_in[to], v[i], u[i]);
                    }
                    if (write_streams) {
                        if constexpr (VEC == 4)
                            *reinterpret_cast<float4*>(xs + (int64_t)to * hidden + c) = make_float4(v[0], v[1], v[2], v[3]);
                        else
                            xs[(int64_t)to * hidden + c] = v[0];
                    }
                }
            }
        } else {
#pragma unroll
            for (int s = 0; s < SMAX; ++s)
                if (s < S) {
#pragma unroll
                    for (int i = 0; i < VEC; ++i) u[i] = fmaf(c_in[s], x[s][i], u[i]);
                }
        }
        if (out != nullptr) {
#pragma unroll
            for (int i = 0; i < VEC; ++i) {
                u_s[c + i] = u[i];
                sq += u[i] * u[i];
            }
        }
    }
    if (out == nullptr) return;
    TO* o = out + r * hidden;
    if (!normalize) {
        for (int c = threadIdx.x * VEC; c < hidden; c += blockDim.x * VEC)     // the thread's own writes
#pragma unroll
            for (int i = 0; i < VEC; ++i) o[c + i] = from_f32<TO>(u_s[c + i]);
        return;
    }
    const float inv = rsqrtf(block_sum(sq, scratch) / (float)hidden + eps);
    for (int c = threadIdx.x * VEC; c < hidden; c += blockDim.x * VEC)
#pragma unroll
        for (int i = 0; i < VEC; ++i) o[c + i] = from_f32<TO>(u_s[c + i] * inv * norm_w[c + i]);
}

template <typename T, typename TO>
int hyper_norm_launch(float* streams, const T* branch, const float* mix, const float* out_coef, const float* in_coef,
                      const float* norm_w, float eps, TO* out, const int* rows, int64_t n_rows, int S, int hidden, int normalize,
                      cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (S <= 0 || S > MAX_STREAMS || hidden <= 0 || n_rows > 0x7fffffffLL) return Q3_ERR_BAD_SIZE;
    if (branch != nullptr && (mix == nullptr || out_coef == nullptr)) return Q3_ERR_BAD_SIZE;
    if (out != nullptr && normalize && norm_w == nullptr) return Q3_ERR_BAD_SIZE;
    const size_t smem = out != nullptr ? (size_t)hidden * sizeof(float) : 0;
    if (smem > 200 * 1024) return Q3_ERR_BAD_SIZE;
    static Q3PerDevice allowed[3];
    const bool vec = hidden % 4 == 0 && aligned16(streams) && S <= 4;
    const bool few = S <= 4;
    if (smem > 48 * 1024) {
        const cudaError_t e = vec   ? q3_allow_shared_memory(hyper_norm_kernel<T, TO, 4, 4>, 200 * 1024, allowed[2])
                              : few ? q3_allow_shared_memory(hyper_norm_kernel<T, TO, 1, 4>, 200 * 1024, allowed[1])
                                    : q3_allow_shared_memory(hyper_norm_kernel<T, TO, 1, MAX_STREAMS>, 200 * 1024, allowed[0]);
        if (e != cudaSuccess) return (int)e;
    }
    const int per = vec ? hidden / 4 : hidden;
    const int threads = per >= 2048 ? 512 : (per >= 512 ? 256 : 128);
    if (vec)
        return (int)q3_launch(hyper_norm_kernel<T, TO, 4, 4>, dim3((unsigned)n_rows), dim3(threads), smem, stream, streams, branch, mix,
                              out_coef, in_coef, norm_w, eps, out, rows, S, hidden, normalize);
    if (few)
        return (int)q3_launch(hyper_norm_kernel<T, TO, 1, 4>, dim3((unsigned)n_rows), dim3(threads), smem, stream, streams, branch, mix,
                              out_coef, in_coef, norm_w, eps, out, rows, S, hidden, normalize);
    return (int)q3_launch(hyper_norm_kernel<T, TO, 1, MAX_STREAMS>, dim3((unsigned)n_rows), dim3(threads), smem, stream, streams, branch,
                          mix, out_coef, in_coef, norm_w, eps, out, rows, S, hidden, normalize);
}

}  // namespace

#define Q3_HYPER_EXPORTS(SUFFIX, T)                                                                                       \
    Q3_EXPORT int q3_embedding_streams_##SUFFIX(const int* ids, const void* table, float* out, int64_t n_tokens, int hidden, \
                                                int vocab, float scale, int copies, void* stream) {                      \
        if (n_tokens <= 0) return 0;                                                                                      \
        if (hidden <= 0 || copies <= 0 || n_tokens > 0x7fffffffLL) return Q3_ERR_BAD_SIZE;                                \
        return (int)q3_launch(embedding_streams_kernel<T>, dim3((unsigned)n_tokens), dim3(hidden >= 1024 ? 256 : 128), 0, \
                              (cudaStream_t)stream, ids, (const T*)table, out, hidden, vocab, scale, copies);             \
    }                                                                                                                     \
    Q3_EXPORT int q3_hyper_norm_##SUFFIX(float* streams, const void* branch, const float* mix, const float* out_coef,     \
                                         const float* in_coef, const float* norm_w, float eps, void* out, int out_f32,    \
                                         const int* rows, int64_t n_rows, int n_streams, int hidden, int normalize,       \
                                         void* stream) {                                                                  \
        if (out_f32)                                                                                                      \
            return hyper_norm_launch<T, float>(streams, (const T*)branch, mix, out_coef, in_coef, norm_w, eps, (float*)out, \
                                               rows, n_rows, n_streams, hidden, normalize, (cudaStream_t)stream);         \
        return hyper_norm_launch<T, T>(streams, (const T*)branch, mix, out_coef, in_coef, norm_w, eps, (T*)out, rows,     \
                                       n_rows, n_streams, hidden, normalize, (cudaStream_t)stream);                       \
    }

Q3_HYPER_EXPORTS(f32, float)
Q3_HYPER_EXPORTS(bf16, bf16)
