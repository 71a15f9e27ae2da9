// Kernels for models whose hidden state between the parts is kept in 32-bit whatever the
// compute type T of the matrix products (float for the 32-bit path, bf16 for serving):
//
//   embedding_scaled : stream[t] = table[ids[t]] * scale                        (T -> float)
//   sandwich_norm    : a branch output y (T) is normalised with weights of its own and added to
//                      the stream, stream += y / rms(y) * w_post, and the sum is normalised for
//                      the next part, out = T(stream / rms(stream) * w_pre): the norm after a
//                      sublayer, the residual sum and the norm before the next sublayer in one
//                      pass over the row.  Either half may be left out (no branch: a plain norm
//                      of the stream; no output: the sum alone).  rms(x) = sqrt(mean(x^2) + eps).
//   concat_cast      : out[t] = T([a[t]; b[t]])  (the input of a product over two streams)
//   gather_rows_norm : rows of the stream picked by index and normalised    (float -> T)
//   scale_softcap    : x <- cap * tanh(x * scale / cap), or x * scale without a cap (float, in place)
//
// Statistics, weights and sums are 32-bit; only `out` is rounded to T.
#include "common.cuh"

namespace {

template <typename T> __device__ __forceinline__ void load4(const T* p, float (&v)[4]);
template <> __device__ __forceinline__ void load4<float>(const float* p, float (&v)[4]) {
    const float4 r = *reinterpret_cast<const float4*>(p);
    v[0] = r.x; v[1] = r.y; v[2] = r.z; v[3] = r.w;
}
template <> __device__ __forceinline__ void load4<bf16>(const bf16* p, float (&v)[4]) {
    const uint2 r = *reinterpret_cast<const uint2*>(p);
    const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&r.x), b = *reinterpret_cast<const __nv_bfloat162*>(&r.y);
    v[0] = __low2float(a); v[1] = __high2float(a); v[2] = __low2float(b); v[3] = __high2float(b);
}
template <typename T> __device__ __forceinline__ void store4(T* p, const float (&v)[4]);
template <> __device__ __forceinline__ void store4<float>(float* p, const float (&v)[4]) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
}
template <> __device__ __forceinline__ void store4<bf16>(bf16* p, const float (&v)[4]) {
    __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
    uint2 r;
    r.x = *reinterpret_cast<uint32_t*>(&a);
    r.y = *reinterpret_cast<uint32_t*>(&b);
    *reinterpret_cast<uint2*>(p) = r;
}

// ---------------------------------------------------------------- embedding * scale
template <typename T>
__global__ void embedding_scaled_kernel(const int* __restrict__ ids, const T* __restrict__ table, float* __restrict__ out,
                                        int hidden, int vocab, float scale) {
    pdl_launch_dependents();
    pdl_wait();
    const int64_t t = blockIdx.x;
    const int id = ids[t];
    const bool ok = id >= 0 && id < vocab;                 // an id outside the table gives a zero row
    const T* src = table + (int64_t)(ok ? id : 0) * hidden;
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) out[t * hidden + c] = ok ? to_f32<T>(src[c]) * scale : 0.0f;
}

// ---------------------------------------------------------------- norm after a branch + sum + norm before the next
// One block per row; a thread keeps PER groups of four values of the row in registers, so the stream is read and
// written once.  PER = 0: any size, the row walked three times through the cache.
template <typename T, int PER>
__global__ void sandwich_norm_kernel(float* __restrict__ stream, const T* __restrict__ branch, const float* __restrict__ w_post,
                                     const float* __restrict__ w_pre, T* __restrict__ out, int size, float eps_post,
                                     float eps_pre) {
    __shared__ float scratch[33];
    pdl_launch_dependents();
    pdl_wait();
    const int64_t row = blockIdx.x;
    float* xr = stream + row * size;
    const T* yr = branch ? branch + row * size : nullptr;
    T* outr = out ? out + row * size : nullptr;
    if constexpr (PER > 0) {
        float x[PER][4], y[PER][4];
        float sq = 0.0f;
#pragma unroll
        for (int p = 0; p < PER; ++p) {
            const int c = (p * blockDim.x + threadIdx.x) * 4;
            if (c < size) {
                load4<float>(xr + c, x[p]);
                if (yr) {
                    load4<T>(yr + c, y[p]);
#pragma unroll
                    for (int i = 0; i < 4; ++i) sq += y[p][i] * y[p][i];
                }
            }
        }
        if (yr) {
            const float inv = rsqrtf(block_sum(sq, scratch) / (float)size + eps_post);
#pragma unroll
            for (int p = 0; p < PER; ++p) {
                const int c = (p * blockDim.x + threadIdx.x) * 4;
                if (c < size) {
                    float w[4];
                    load4<float>(w_post + c, w);
#pragma unroll
                    for (int i = 0; i < 4; ++i) x[p][i] += y[p][i] * inv * w[i];
                    store4<float>(xr + c, x[p]);
                }
            }
        }
        if (outr == nullptr) return;
        sq = 0.0f;
#pragma unroll
        for (int p = 0; p < PER; ++p) {
            const int c = (p * blockDim.x + threadIdx.x) * 4;
            if (c < size) {
#pragma unroll
                for (int i = 0; i < 4; ++i) sq += x[p][i] * x[p][i];
            }
        }
        const float inv = rsqrtf(block_sum(sq, scratch) / (float)size + eps_pre);
#pragma unroll
        for (int p = 0; p < PER; ++p) {
            const int c = (p * blockDim.x + threadIdx.x) * 4;
            if (c < size) {
                float w[4], v[4];
                load4<float>(w_pre + c, w);
#pragma unroll
                for (int i = 0; i < 4; ++i) v[i] = x[p][i] * inv * w[i];
                store4<T>(outr + c, v);
            }
        }
    } else {
        if (yr) {
            float sq = 0.0f;
            for (int c = threadIdx.x; c < size; c += blockDim.x) {
                const float v = to_f32<T>(yr[c]);
                sq += v * v;
            }
            const float inv = rsqrtf(block_sum(sq, scratch) / (float)size + eps_post);
            for (int c = threadIdx.x; c < size; c += blockDim.x) xr[c] += to_f32<T>(yr[c]) * inv * w_post[c];
        }
        if (outr == nullptr) return;
        float sq = 0.0f;
        for (int c = threadIdx.x; c < size; c += blockDim.x) sq += xr[c] * xr[c];       // the thread's own writes
        const float inv = rsqrtf(block_sum(sq, scratch) / (float)size + eps_pre);
        for (int c = threadIdx.x; c < size; c += blockDim.x) outr[c] = from_f32<T>(xr[c] * inv * w_pre[c]);
    }
}

template <typename T>
int sandwich_norm_launch(float* stream, const T* branch, const float* w_post, const float* w_pre, T* out, int64_t rows, int size,
                         float eps_post, float eps_pre, cudaStream_t s) {
    if (rows <= 0) return 0;
    if (size <= 0 || (branch != nullptr) != (w_post != nullptr) || (out != nullptr) != (w_pre != nullptr)) return Q3_ERR_BAD_SIZE;
    if (rows > 0x7fffffffLL) return Q3_ERR_TOO_LARGE;
    const bool vec = size % 4 == 0 && aligned16(stream) && (branch == nullptr || aligned16(branch)) && (out == nullptr || aligned16(out)) &&
                     (w_post == nullptr || aligned16(w_post)) && (w_pre == nullptr || aligned16(w_pre));
    const int groups = size / 4;
    auto launch = [&](auto kernel, int threads) {
        return (int)q3_launch(kernel, dim3((unsigned)rows), dim3(threads), 0, s, stream, branch, w_post, w_pre, out, size, eps_post, eps_pre);
    };
    if (vec && groups <= 2048) {
        const int per = groups <= 256 ? 1 : (groups <= 512 ? 2 : (groups <= 1024 ? 4 : 8));
        const int threads = ((groups + per - 1) / per + 31) / 32 * 32;
        if (per == 1) return launch(sandwich_norm_kernel<T, 1>, threads);
        if (per == 2) return launch(sandwich_norm_kernel<T, 2>, threads);
        if (per == 4) return launch(sandwich_norm_kernel<T, 4>, threads);
        return launch(sandwich_norm_kernel<T, 8>, threads);
    }
    return launch(sandwich_norm_kernel<T, 0>, size >= 1024 ? 512 : 128);
}

// ---------------------------------------------------------------- [a; b] in the compute type
// Four values a thread where the rows allow 16-byte reads.
template <typename T>
__global__ void concat_cast_vec_kernel(const float* __restrict__ a, const float* __restrict__ b, T* __restrict__ out, int64_t rows,
                                       int size) {
    pdl_launch_dependents();
    pdl_wait();
    const int groups = size / 4;
    const int64_t total = rows * 2 * groups;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = i / (2 * groups);
        const int g = (int)(i % (2 * groups));
        float v[4];
        load4<float>((g < groups ? a + r * size : b + r * size - size) + 4 * g, v);
        store4<T>(out + r * 2 * size + 4 * g, v);
    }
}

template <typename T>
__global__ void concat_cast_kernel(const float* __restrict__ a, const float* __restrict__ b, T* __restrict__ out, int64_t rows,
                                   int size) {
    pdl_launch_dependents();
    pdl_wait();
    const int64_t total = rows * 2 * size;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = i / (2 * size);
        const int c = (int)(i % (2 * size));
        out[i] = from_f32<T>(c < size ? a[r * size + c] : b[r * size + c - size]);
    }
}

// ---------------------------------------------------------------- picked rows, normalised
template <typename T>
__global__ void gather_rows_norm_kernel(const float* __restrict__ stream, const int* __restrict__ idx, const float* __restrict__ w,
                                        T* __restrict__ out, int size, float eps) {
    __shared__ float scratch[33];
    pdl_launch_dependents();
    pdl_wait();
    const float* xr = stream + (int64_t)idx[blockIdx.x] * size;
    float sq = 0.0f;
    for (int c = threadIdx.x; c < size; c += blockDim.x) sq += xr[c] * xr[c];
    const float inv = rsqrtf(block_sum(sq, scratch) / (float)size + eps);
    for (int c = threadIdx.x; c < size; c += blockDim.x) out[(int64_t)blockIdx.x * size + c] = from_f32<T>(xr[c] * inv * w[c]);
}

// ---------------------------------------------------------------- scale and smooth cap, in place
__global__ void scale_softcap_kernel(float* __restrict__ x, int64_t n, float scale, float cap) {
    pdl_launch_dependents();
    pdl_wait();
    const float inv = cap > 0.0f ? 1.0f / cap : 0.0f;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        const float v = x[i] * scale;
        x[i] = cap > 0.0f ? cap * tanhf(v * inv) : v;
    }
}

static unsigned grid_for(int64_t work, int threads) {
    int64_t blocks = (work + threads - 1) / threads;
    const int64_t resident = (int64_t)q3_device_sm_count() * 8;
    return (unsigned)(blocks > resident ? resident : (blocks < 1 ? 1 : blocks));
}

}  // namespace

#define Q3_STREAM_EXPORTS(SUFFIX, T)                                                                                     \
    Q3_EXPORT int q3_embedding_scaled_##SUFFIX(const int* ids, const void* table, float* out, int64_t n_tokens, int hidden, \
                                               int vocab, float scale, void* stream) {                                  \
        if (n_tokens <= 0) return 0;                                                                                     \
        if (hidden <= 0 || n_tokens > 0x7fffffffLL) return Q3_ERR_BAD_SIZE;                                              \
        return (int)q3_launch(embedding_scaled_kernel<T>, dim3((unsigned)n_tokens), dim3(hidden >= 1024 ? 256 : 128), 0, \
                              (cudaStream_t)stream, ids, (const T*)table, out, hidden, vocab, scale);                    \
    }                                                                                                                    \
    Q3_EXPORT int q3_sandwich_norm_##SUFFIX(float* stream_rows, const void* branch, const float* w_post, const float* w_pre, \
                                            void* out, int64_t rows, int size, float eps_post, float eps_pre,           \
                                            void* stream) {                                                              \
        return sandwich_norm_launch<T>(stream_rows, (const T*)branch, w_post, w_pre, (T*)out, rows, size, eps_post,      \
                                       eps_pre, (cudaStream_t)stream);                                                   \
    }                                                                                                                    \
    Q3_EXPORT int q3_concat_cast_##SUFFIX(const float* a, const float* b, void* out, int64_t rows, int size, void* stream) { \
        if (rows <= 0) return 0;                                                                                         \
        if (size <= 0) return Q3_ERR_BAD_SIZE;                                                                           \
        if (size % 4 == 0 && aligned16(a) && aligned16(b) && aligned16(out))                                             \
            return (int)q3_launch(concat_cast_vec_kernel<T>, dim3(grid_for(rows * 2 * (size / 4), 256)), dim3(256), 0,   \
                                  (cudaStream_t)stream, a, b, (T*)out, rows, size);                                      \
        return (int)q3_launch(concat_cast_kernel<T>, dim3(grid_for(rows * 2 * size, 256)), dim3(256), 0,                 \
                              (cudaStream_t)stream, a, b, (T*)out, rows, size);                                          \
    }                                                                                                                    \
    Q3_EXPORT int q3_gather_rows_norm_##SUFFIX(const float* stream_rows, const int* idx, const float* w, void* out,      \
                                               int64_t rows, int size, float eps, void* stream) {                        \
        if (rows <= 0) return 0;                                                                                         \
        if (size <= 0 || rows > 0x7fffffffLL) return Q3_ERR_BAD_SIZE;                                                    \
        return (int)q3_launch(gather_rows_norm_kernel<T>, dim3((unsigned)rows), dim3(size >= 1024 ? 256 : 128), 0,       \
                              (cudaStream_t)stream, stream_rows, idx, w, (T*)out, size, eps);                            \
    }

Q3_STREAM_EXPORTS(f32, float)
Q3_STREAM_EXPORTS(bf16, bf16)

Q3_EXPORT int q3_scale_softcap_f32(float* x, int64_t n, float scale, float cap, void* stream) {
    if (n <= 0) return 0;
    return (int)q3_launch(scale_softcap_kernel, dim3(grid_for(n, 256)), dim3(256), 0, (cudaStream_t)stream, x, n, scale, cap);
}
