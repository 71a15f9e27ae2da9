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
//   lightning_chunks_tc : the chunked form with its four products per chunk on the tensor cores (namespace tc below).
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

// ---------------------------------------------------------------- the chunks' products on the tensor cores
// The same four products per chunk of C = 32 tokens as above,
//     A = (Q K^T) o decay^(i-j)      inter = Q S_0      o = decay^(i+1) inter + A V      S <- decay^C S_0 + (decay^(C-1-j) K)^T V,
// as tiles of mma.m16n8k8 with 32-bit operands: every operand is split into its TF32 rounding and what that dropped (hi + lo),
// and a product is three instructions (lo x hi, hi x lo, hi x hi) accumulated in 32-bit, which keeps about 21 bits of every
// factor - well beyond what a compute type of bfloat16 asks of a 32-bit recurrence, and it is used for that compute type only
// (the float32 path stays on fmaf).  A block of 8 warps per (head, sequence, tile of `vt` state columns) keeps q, k (C x d), its
// columns of v, the C x C scores and its share of the state, d x vt, in shared memory; head sizes in steps of 8.
namespace tc {
constexpr int C = 32;

__device__ __forceinline__ void split_tf32(float x, uint32_t& hi, uint32_t& lo) {
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(hi) : "f"(x));
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(lo) : "f"(x - __uint_as_float(hi)));
}
__device__ __forceinline__ void mma_tf32(float (&c)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
    asm volatile("mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

// c[16 x 8] += A[16 x K] B[K x 8].  A(m, k) lies at A[m * lda + k] (A_T: at A[k * lda + m]), B(k, n) at B[k * ldb + n]
// (B_NK: at B[n * ldb + k]); `k_scale` (may be null) multiplies column k of A.  Fragments of m16n8k8: a0 (g, t), a1 (g + 8, t),
// a2 (g, t + 4), a3 (g + 8, t + 4); b0 (t, g), b1 (t + 4, g); c0 (g, 2t), c1 (g, 2t + 1), c2 (g + 8, 2t), c3 (g + 8, 2t + 1).
template <bool A_T, bool B_NK>
__device__ __forceinline__ void tile(float (&c)[4], const float* A, int lda, const float* B, int ldb, int K, int lane,
                                     const float* k_scale) {
    const int g = lane >> 2, t = lane & 3;
    for (int k0 = 0; k0 < K; k0 += 8) {
        float a[4], b[2];
        if (A_T) {
            a[0] = A[(k0 + t) * lda + g];     a[1] = A[(k0 + t) * lda + g + 8];
            a[2] = A[(k0 + t + 4) * lda + g]; a[3] = A[(k0 + t + 4) * lda + g + 8];
        } else {
            a[0] = A[g * lda + k0 + t];       a[1] = A[(g + 8) * lda + k0 + t];
            a[2] = A[g * lda + k0 + t + 4];   a[3] = A[(g + 8) * lda + k0 + t + 4];
        }
        if (k_scale != nullptr) {
            const float s0 = k_scale[k0 + t], s1 = k_scale[k0 + t + 4];
            a[0] *= s0; a[1] *= s0; a[2] *= s1; a[3] *= s1;
        }
        if (B_NK) {
            b[0] = B[g * ldb + k0 + t];       b[1] = B[g * ldb + k0 + t + 4];
        } else {
            b[0] = B[(k0 + t) * ldb + g];     b[1] = B[(k0 + t + 4) * ldb + g];
        }
        uint32_t ah[4], al[4], bh[2], bl[2];
#pragma unroll
        for (int i = 0; i < 4; ++i) split_tf32(a[i], ah[i], al[i]);
#pragma unroll
        for (int i = 0; i < 2; ++i) split_tf32(b[i], bh[i], bl[i]);
        mma_tf32(c, al, bh);
        mma_tf32(c, ah, bl);
        mma_tf32(c, ah, bh);
    }
}

template <typename T>
__global__ void __launch_bounds__(256)
lightning_chunks_tc_kernel(const T* __restrict__ proj, float* __restrict__ state, const float* __restrict__ decay,
                           const int* __restrict__ seq_start, const int* __restrict__ seq_slots, float* __restrict__ out, int H, int d,
                           int vd, int vt) {
    extern __shared__ float smem[];
    const int dp = (d + 15) & ~15;                      // rows of the state in whole 16-row tiles; the padding stays zero
    const int ldq = dp + 4, ldv = vt + 8, lda = C + 4;  // row lengths that spread the fragments' rows over the banks
    float* q_s = smem;                                  // [C][ldq]
    float* k_s = q_s + C * ldq;                         // [C][ldq]
    float* v_s = k_s + C * ldq;                         // [C][ldv]
    float* a_s = v_s + C * ldv;                         // [C][lda]
    float* S_s = a_s + C * lda;                         // [dp][ldv]
    __shared__ float pw[C + 1], pw_rev[C];
    pdl_launch_dependents();
    pdl_wait();
    const int head = blockIdx.x, seq = blockIdx.y, col0 = blockIdx.z * vt;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const float lam = decay[head];
    const float l2 = lam > 0.0f ? log2f(lam) : 0.0f;
    for (int n = tid; n <= C; n += 256) pw[n] = n == 0 ? 1.0f : (lam > 0.0f ? exp2f((float)n * l2) : 0.0f);
    const int64_t cols = 2 * (int64_t)H * d + 2 * (int64_t)H * vd;
    float* S_g = state + ((int64_t)seq_slots[seq] * H + head) * d * vd;
    for (int x = tid; x < dp * ldv; x += 256) {
        const int i = x / ldv, c = x % ldv;
        S_s[x] = (i < d && c < vt && col0 + c < vd) ? S_g[(int64_t)i * vd + col0 + c] : 0.0f;
    }
    for (int x = tid; x < 2 * C * ldq + C * ldv; x += 256) smem[x] = 0.0f;     // the padding of q, k and v stays zero
    const int n_tiles = vt / 8;                          // 8-column tiles of this block's state columns
    const int t_end = seq_start[seq + 1];
    for (int t0 = seq_start[seq]; t0 < t_end; t0 += C) {
        const int Cn = min(C, t_end - t0);
        __syncthreads();                                 // the chunk before is done with the buffers; S_s holds its state
        // 16-byte packets of the projection's rows (head sizes are multiples of 8); rows beyond the chunk are zero
        constexpr int VEC = Pack<T>::N;
        for (int x = tid; x < C * (d / VEC); x += 256) {
            const int i = x / (d / VEC), c = x % (d / VEC) * VEC;
            float qv[VEC], kv[VEC];
            if (i < Cn) {
                const T* row = proj + (int64_t)(t0 + i) * cols;
                const Pack<T> qp = load_pack<T>(row + (int64_t)head * d + c), kp = load_pack<T>(row + (int64_t)(H + head) * d + c);
#pragma unroll
                for (int e = 0; e < VEC; ++e) {
                    qv[e] = silu_f32(qp.get(e));
                    kv[e] = silu_f32(kp.get(e));
                }
            } else {
#pragma unroll
                for (int e = 0; e < VEC; ++e) qv[e] = kv[e] = 0.0f;
            }
#pragma unroll
            for (int e = 0; e < VEC; ++e) {
                q_s[i * ldq + c + e] = qv[e];
                k_s[i * ldq + c + e] = kv[e];
            }
        }
        for (int x = tid; x < C * (vt / VEC); x += 256) {
            const int i = x / (vt / VEC), c = x % (vt / VEC) * VEC;
            float vv[VEC];
#pragma unroll
            for (int e = 0; e < VEC; ++e) vv[e] = 0.0f;
            if (i < Cn && col0 + c < vd) {
                const Pack<T> vp = load_pack<T>(proj + (int64_t)(t0 + i) * cols + 2 * (int64_t)H * d + (int64_t)head * vd + col0 + c);
#pragma unroll
                for (int e = 0; e < VEC; ++e) vv[e] = silu_f32(vp.get(e));
            }
#pragma unroll
            for (int e = 0; e < VEC; ++e) v_s[i * ldv + c + e] = vv[e];
        }
        if (tid < C) pw_rev[tid] = tid < Cn ? pw[Cn - 1 - tid] : 0.0f;
        __syncthreads();
        // the scores of the chunk: 2 x 4 tiles of 16 x 8, one per warp
        {
            const int mi = warp & 1, ni = warp >> 1;
            float c4[4] = {0.0f, 0.0f, 0.0f, 0.0f};
            tile<false, true>(c4, q_s + mi * 16 * ldq, ldq, k_s + ni * 8 * ldq, ldq, dp, lane, nullptr);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int i = mi * 16 + g + (e >> 1) * 8, j = ni * 8 + 2 * t + (e & 1);
                a_s[i * lda + j] = j <= i ? c4[e] * pw[i - j] : 0.0f;
            }
        }
        // what the state before the chunk gives every token: this warp's 16 rows (warp & 1) and every fourth column tile
        const int mi = warp & 1;
        float inter[8][4];                               // up to 8 column tiles a warp (vt <= 256)
#pragma unroll
        for (int n = 0; n < 8; ++n) {
            inter[n][0] = inter[n][1] = inter[n][2] = inter[n][3] = 0.0f;
            const int ni = (warp >> 1) + 4 * n;
            if (ni < n_tiles) tile<false, false>(inter[n], q_s + mi * 16 * ldq, ldq, S_s + ni * 8, ldv, dp, lane, nullptr);
        }
        __syncthreads();                                 // the scores are written; every warp has read the old state
#pragma unroll
        for (int n = 0; n < 8; ++n) {
            const int ni = (warp >> 1) + 4 * n;
            if (ni < n_tiles) {
                float intra[4] = {0.0f, 0.0f, 0.0f, 0.0f};
                tile<false, false>(intra, a_s + mi * 16 * lda, lda, v_s + ni * 8, ldv, C, lane, nullptr);
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int i = mi * 16 + g + (e >> 1) * 8, c = col0 + ni * 8 + 2 * t + (e & 1);
                    if (i < Cn && c < vd) out[((int64_t)(t0 + i) * H + head) * vd + c] = fmaf(pw[i + 1], inter[n][e], intra[e]);
                }
            }
        }
        // the state after the chunk: 16-row tiles of the state dealt to the warps
        for (int mt = warp; mt < dp / 16; mt += 8) {
            for (int ni = 0; ni < n_tiles; ++ni) {
                float* Sp = S_s + (mt * 16) * ldv + ni * 8;
                float c4[4];
                c4[0] = Sp[g * ldv + 2 * t] * pw[Cn];       c4[1] = Sp[g * ldv + 2 * t + 1] * pw[Cn];
                c4[2] = Sp[(g + 8) * ldv + 2 * t] * pw[Cn]; c4[3] = Sp[(g + 8) * ldv + 2 * t + 1] * pw[Cn];
                tile<true, false>(c4, k_s + mt * 16, ldq, v_s + ni * 8, ldv, C, lane, pw_rev);
                Sp[g * ldv + 2 * t] = c4[0];       Sp[g * ldv + 2 * t + 1] = c4[1];
                Sp[(g + 8) * ldv + 2 * t] = c4[2]; Sp[(g + 8) * ldv + 2 * t + 1] = c4[3];
            }
        }
    }
    __syncthreads();
    for (int x = tid; x < d * vt; x += 256) {
        const int i = x / vt, c = x % vt;
        if (col0 + c < vd) S_g[(int64_t)i * vd + col0 + c] = S_s[i * ldv + c];
    }
}

static inline size_t smem_bytes(int d, int vt) {
    const int dp = (d + 15) & ~15;
    return (size_t)(2 * C * (dp + 4) + C * (vt + 8) + C * (C + 4) + dp * (vt + 8)) * sizeof(float);
}

template <typename T>
int launch(const T* proj, float* state, const float* decay, const int* seq_start, const int* seq_slots, float* out, int n_seqs, int H,
           int d, int vd, cudaStream_t stream) {
    if (n_seqs <= 0) return 0;
    if (H <= 0 || d <= 0 || vd <= 0 || d > 256 || vd > 256 || d % 8 != 0 || vd % 8 != 0 || n_seqs > 65535) return Q3_ERR_BAD_SIZE;
    if (!aligned16(proj)) return Q3_ERR_MISALIGNED;
    // as many state columns a block as keep the multiprocessors busy: 64, or 32 / 16 while the blocks are too few (measured on
    // one prompt of 2,048 tokens with 16 heads of 128 x 128: 1.03 ms with 64 columns, 0.77 with 32, 0.63 with 16, 0.76 with 8)
    int vt = min(vd, 64);
    while (vt > 16 && vt % 16 == 0 && (int64_t)H * n_seqs * ((vd + vt - 1) / vt) < q3_device_sm_count()) vt /= 2;
    const size_t smem = smem_bytes(d, vt);
    if (smem > 200 * 1024) return Q3_ERR_BAD_SIZE;
    static Q3PerDevice allowed;
    const cudaError_t e = q3_allow_shared_memory(lightning_chunks_tc_kernel<T>, 200 * 1024, allowed);
    if (e != cudaSuccess) return (int)e;
    return (int)q3_launch(lightning_chunks_tc_kernel<T>, dim3(H, n_seqs, (vd + vt - 1) / vt), dim3(256), smem, stream, proj, state, decay,
                          seq_start, seq_slots, out, H, d, vd, vt);
}
}  // namespace tc

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

// The chunked form with its products on the tensor cores (operands split into TF32 hi + lo terms): for a compute type of
// bfloat16, head sizes in steps of 8.
Q3_EXPORT int q3_lightning_chunks_tc_bf16(const void* proj, float* state, const float* decay, const int* seq_start,
                                          const int* seq_slots, float* out, int n_seqs, int heads, int d, int vd, void* stream) {
    return tc::launch<bf16>((const bf16*)proj, state, decay, seq_start, seq_slots, out, n_seqs, heads, d, vd, (cudaStream_t)stream);
}

Q3_LIGHTNING_EXPORTS(f32, float)
Q3_LIGHTNING_EXPORTS(bf16, bf16)
