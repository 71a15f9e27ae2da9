// Differential attention: every head has two softmax maps over the same values, and its output is their
// weighted difference, brought to unit rms:
//
//     o = a1 - lambda a2;   out = o / sqrt(mean(o^2) + eps) * gain        (per token and head, over vd values)
//
//   diff_combine : a [token, group, map, head in group, vd] float32 (the two maps' outputs, laid out as the
//                  attention kernels see their query heads: the heads of a key head side by side) ->
//                  out [token, head, vd] in the compute type T.  One warp per (token, head); 32-bit throughout.
#include "common.cuh"

namespace {

template <typename T>
__global__ void diff_combine_kernel(const float* __restrict__ a, T* __restrict__ out, int64_t n_tokens, int heads, int per_group,
                                    int vd, float lambda, float eps, float gain) {
    pdl_launch_dependents();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const int64_t item = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (item >= n_tokens * heads) return;
    const int64_t t = item / heads;
    const int head = (int)(item % heads), g = head / per_group, hh = head % per_group;
    const float* a1 = a + ((t * (heads / per_group) + g) * 2 * per_group + hh) * (int64_t)vd;
    const float* a2 = a1 + (int64_t)per_group * vd;
    float o[8];                                            // vd <= 256
    float sq = 0.0f;
#pragma unroll
    for (int n = 0; n < 8; ++n) {
        const int c = lane + 32 * n;
        o[n] = c < vd ? a1[c] - lambda * a2[c] : 0.0f;
        sq += o[n] * o[n];
    }
    const float inv = rsqrtf(warp_sum(sq) / (float)vd + eps) * gain;
    T* dst = out + item * vd;
#pragma unroll
    for (int n = 0; n < 8; ++n) {
        const int c = lane + 32 * n;
        if (c < vd) dst[c] = from_f32<T>(o[n] * inv);
    }
}

}  // namespace

#define Q3_DIFFERENTIAL_EXPORTS(SUFFIX, T)                                                                               \
    Q3_EXPORT int q3_diff_combine_##SUFFIX(const float* a, void* out, int64_t n_tokens, int heads, int per_group, int vd, \
                                           float lambda, float eps, float gain, void* stream) {                          \
        if (n_tokens <= 0) return 0;                                                                                     \
        if (heads <= 0 || per_group <= 0 || heads % per_group != 0 || vd <= 0 || vd > 256) return Q3_ERR_BAD_SIZE;       \
        const int64_t blocks = (n_tokens * heads + 3) / 4;                                                               \
        if (blocks > 0x7fffffffLL) return Q3_ERR_TOO_LARGE;                                                              \
        return (int)q3_launch(diff_combine_kernel<T>, dim3((unsigned)blocks), dim3(128), 0, (cudaStream_t)stream, a,     \
                              (T*)out, n_tokens, heads, per_group, vd, lambda, eps, gain);                               \
    }

Q3_DIFFERENTIAL_EXPORTS(f32, float)
Q3_DIFFERENTIAL_EXPORTS(bf16, bf16)
