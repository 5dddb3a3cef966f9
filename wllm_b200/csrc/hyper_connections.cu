// A residual kept as S streams x_1 .. x_S [S][n][H] (32-bit) that sublayers read and write through learned weights,
// and the root-mean-square norm in front of a sublayer, in ONE kernel a sublayer:
//
//   (1) the sublayer before left its output y pending (a tensor, or `parts` partial sums added in order), with the
//       weights of its connection: every stream becomes, all at once from the old ones,
//           x_t <- sum_s mix[s][t] * x_s + out[t] * y                     (written back, unless `rows` is given)
//   (2) the input of this sublayer is u = sum_s in[s] * x_s (in = null: the plain sum of the streams, which is
//       what the model's last norm reads), and   normed = u / sqrt(mean(u^2) + eps) * gain.
//
// Without a pending output step (1) is left out.  The streams may be read from one place and written to another
// (`src_stride` 0: all S streams are read from the same rows, which is how the first norm of a model spreads the
// embedding's output over the streams).  With `rows` the kernel reads row rows[i], writes the normed row i and
// leaves the streams as they are.  All arithmetic is 32-bit in an order that depends on nothing but the row: sums over s
// ascend, and the sum of squares is that of 1,024 lanes (lane c mod 1,024 takes column c, in ascending order; the lanes of
// every 32 are added by the xor tree, the 32 groups in order) whatever the number of threads: a CTA of 1,024 / A threads
// keeps A of those lanes a thread.  So few rows (a decode step) run a thread a column or two, with every load of a row in
// flight at once (33 -> 6 us a launch at 8 rows of 2,048 with 9 partial sums), many rows run CTAs of 256 threads, and both
// give the same bits.  One block a row; u waits in shared memory between the two passes.
#include "common.cuh"

constexpr int HC_MAX_STREAMS = 16;

template <typename TD>
__device__ __forceinline__ float pending_sum(const TD* __restrict__ d, int parts, size_t stride) {
    if (parts == 1) return to_f32(d[0]);
    float v = 0.f;
    for (int sp = 0; sp < parts; sp += 16) {      // sixteen loads in flight; the additions are in order
        float part[16];
#pragma unroll
        for (int u = 0; u < 16; ++u) part[u] = sp + u < parts ? to_f32(d[(size_t)(sp + u) * stride]) : 0.f;
#pragma unroll
        for (int u = 0; u < 16; ++u)
            if (sp + u < parts) v = (sp + u == 0) ? part[u] : v + part[u];
    }
    return v;
}

template <typename TD, typename TO, int S_FIXED, int A>   // S_FIXED > 0: that many streams, loops unrolled; 0: any number up to the limit
__global__ void __launch_bounds__(1024)
hyper_norm_kernel(const float* __restrict__ src, size_t src_stride, float* __restrict__ dst, size_t dst_stride, int S_any,
                  const TD* __restrict__ delta, int parts, size_t part_stride, const float* __restrict__ prev_mix,
                  const float* __restrict__ prev_out, const float* __restrict__ in_w, const float* __restrict__ gain,
                  float eps, TO* __restrict__ out, const int* __restrict__ rows, int H) {
    extern __shared__ float u_smem[];
    __shared__ float scratch[32];
    __shared__ float w_mix[HC_MAX_STREAMS * HC_MAX_STREAMS], w_out[HC_MAX_STREAMS], w_in[HC_MAX_STREAMS];
    pdl_launch_dependents();
    const int S = S_FIXED > 0 ? S_FIXED : S_any;
    // the connection weights are written by no kernel of a step: read before the wait
    for (int i = threadIdx.x; i < S * S; i += blockDim.x) w_mix[i] = prev_mix ? prev_mix[i] : 0.f;
    for (int i = threadIdx.x; i < S; i += blockDim.x) {
        w_out[i] = prev_out ? prev_out[i] : 0.f;
        w_in[i] = in_w ? in_w[i] : 1.0f;
    }
    __syncthreads();
    pdl_wait();
    const int i = blockIdx.x;
    const int row = rows ? rows[i] : i;
    const bool update = delta != nullptr;
    const bool write_back = rows == nullptr && (update || dst != src || src_stride != dst_stride);
    constexpr int SR = S_FIXED > 0 ? S_FIXED : HC_MAX_STREAMS;
    constexpr int UF = S_FIXED > 0 ? S_FIXED : 1;       // any number of streams: loops as they are, x[] on the stack
    float ssv[A];
#pragma unroll
    for (int a = 0; a < A; ++a) ssv[a] = 0.f;
    for (int c0 = threadIdx.x; c0 < H; c0 += 1024)
#pragma unroll
    for (int a = 0; a < A; ++a) {
        const int c = c0 + a * (1024 / A);
        if (c >= H) break;
        float x[SR];
#pragma unroll UF
        for (int s = 0; s < SR; ++s) x[s] = s < S ? src[(size_t)s * src_stride + (size_t)row * H + c] : 0.f;
        float u = 0.f;
        if (update) {
            const float y = pending_sum<TD>(delta + (size_t)row * H + c, parts, part_stride);
#pragma unroll UF
            for (int t = 0; t < SR; ++t) {
                if (t >= S) break;
                float acc = 0.f;
#pragma unroll UF
                for (int s = 0; s < SR; ++s)
                    if (s < S) acc = s == 0 ? __fmul_rn(w_mix[t], x[0]) : fmaf(w_mix[s * S + t], x[s], acc);
                acc = fmaf(w_out[t], y, acc);
                if (write_back) dst[(size_t)t * dst_stride + (size_t)row * H + c] = acc;
                u = t == 0 ? __fmul_rn(w_in[0], acc) : fmaf(w_in[t], acc, u);
            }
        } else {
#pragma unroll UF
            for (int t = 0; t < SR; ++t) {
                if (t >= S) break;
                if (write_back) dst[(size_t)t * dst_stride + (size_t)row * H + c] = x[t];
                u = t == 0 ? __fmul_rn(w_in[0], x[0]) : fmaf(w_in[t], x[t], u);
            }
        }
        u_smem[c] = u;
        ssv[a] = fmaf(u, u, ssv[a]);
    }
    // lanes 32 g .. 32 g + 31 of the 1,024 are accumulator g / (warps) of warp g % (warps): their tree, then the groups in order
    __syncthreads();
#pragma unroll
    for (int a = 0; a < A; ++a) {
        const float v = warp_sum(ssv[a]);
        if ((threadIdx.x & 31) == 0) scratch[a * (32 / A) + (threadIdx.x >> 5)] = v;
    }
    __syncthreads();
    float ss = 0.f;
    for (int g = 0; g < 32; ++g) ss += scratch[g];
    const float inv = 1.0f / sqrtf(ss / (float)H + eps);
    TO* o = out + (size_t)i * H;
    for (int c = threadIdx.x; c < H; c += blockDim.x) o[c] = from_f32<TO>((u_smem[c] * inv) * gain[c]);
}

// src: [S][n][H] (or one [n][H] read by every stream with src_stride 0); dst likewise (may be src); delta: the pending
// sublayer output [n][H] of delta_dtype, or `parts` 32-bit partial sums `part_stride` elements apart, or null;
// prev_mix [S][S] indexed [from][to], prev_out [S]: the connection of the sublayer that left delta; in_w [S] or null
// (plain sum); gain [H] 32-bit; rows: null or n_out row indices.
WLLM_API int wllm_hyper_norm(const float* src, long long src_stride, float* dst, long long dst_stride, int S,
                             const void* delta, int delta_dtype, int parts, long long part_stride, const float* prev_mix,
                             const float* prev_out, const float* in_w, const float* gain, float eps, void* out,
                             int out_dtype, const int* rows, int n_out, int H, cudaStream_t stream) {
    if (n_out <= 0) return WLLM_OK;
    if (S < 1 || S > HC_MAX_STREAMS || H <= 0 || parts < 1 || (size_t)H * sizeof(float) > 200 * 1024) return WLLM_BAD_SIZE;
    if (delta != nullptr && (prev_mix == nullptr || prev_out == nullptr)) return WLLM_BAD_SIZE;
    if (delta != nullptr && parts > 1 && delta_dtype != WLLM_F32) return WLLM_BAD_DTYPE;
    const size_t smem = (size_t)H * sizeof(float);
    const bool few = n_out <= 64 && H >= 1024;           // see the kernel's text: the bits do not depend on this choice
#define GO4(TD, TO, SF, AA) do { \
        if (smem > 48 * 1024) { \
            const cudaError_t e = cudaFuncSetAttribute(hyper_norm_kernel<TD, TO, SF, AA>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024); \
            if (e != cudaSuccess) return 1000 + (int)e; \
        } \
        return wllm_launch(hyper_norm_kernel<TD, TO, SF, AA>, n_out, 1024 / AA, smem, stream, src, (size_t)src_stride, dst, \
                           (size_t)dst_stride, S, (const TD*)delta, parts, (size_t)part_stride, prev_mix, prev_out, in_w, gain, \
                           eps, (TO*)out, rows, H); \
    } while (0)
#define GO3(TD, TO, SF) do { if (few) GO4(TD, TO, SF, 1); if (H >= 1024) GO4(TD, TO, SF, 4); GO4(TD, TO, SF, 8); } while (0)
#define GO(TD, TO) do { if (S == 1) GO3(TD, TO, 1); if (S == 2) GO3(TD, TO, 2); if (S == 4) GO3(TD, TO, 4); GO3(TD, TO, 0); } while (0)
    const bool d32 = delta == nullptr || delta_dtype == WLLM_F32;
    if (!d32 && delta_dtype != WLLM_BF16) return WLLM_BAD_DTYPE;
    if (out_dtype == WLLM_BF16) { if (d32) GO(float, bf16); GO(bf16, bf16); }
    if (out_dtype == WLLM_F32) { if (d32) GO(float, float); GO(bf16, float); }
#undef GO
#undef GO3
#undef GO4
    return WLLM_BAD_DTYPE;
}
