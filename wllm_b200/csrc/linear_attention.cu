// Linear attention with a decayed matrix state per (request, head):
//
//     S_t = diag(a_t) S_(t-1) + k_t v_t^T          S: [dim, vdim], 32-bit, one per request and head
//     o_t = S_t^T q_t
//
// a_t is a decay per key channel and token (gated linear attention) or one constant per head (retention).
// The state lives in the cache manager's state slots and is carried from step to step; a request's tokens of
// one step are walked in order from the state that the step before left, so a whole prompt, a portion and a
// single decoded token are one case and give the same bits.
//
// Three entry points, all 32-bit inside:
//   wllm_linattn_prepare    from a fused projection row (q | k | v | ... in one matrix product, possibly still in
//                           split-K slabs): q and k turned by the rotary angle of the token's position (optional),
//                           scaled, v copied, and the decay of every key channel worked out from a low-rank map:
//                               z = W2 (x W1^T) + b,   a = sigmoid(z)^(1/tau) = exp(log_sigmoid(z) / tau)
//   wllm_linattn_scan       the recurrence.  Grid (tiles of 64 value columns, heads, requests); a lane owns two
//                           columns of S, a warp a run of at most 16 key channels of them, in registers.  Tokens
//                           arrive in tiles of 8 through a two-stage cp.async ring; the warps' partial dot products of a
//                           tile's tokens meet in shared memory once a tile and are added in warp order.  Long portions of prompts are cut
//                           into segments that are walked side by side: from zero for their local end states, which a
//                           small kernel chains into start states, and once more from those for the outputs.
//   wllm_head_gate_norm     per head: o / sqrt(mean(o^2) + eps) [* w] * silu(g), rounded once to the matrix type
//                           (the operand of the output projection).
#include "common.cuh"

__device__ __forceinline__ float la_any(const void* p, int dtype, size_t i) {
    return dtype == WLLM_BF16 ? __bfloat162float(reinterpret_cast<const bf16*>(p)[i]) : reinterpret_cast<const float*>(p)[i];
}
// element i of a row that may come as `parts` slabs `stride` elements apart, added in slab order
// (several parts are always 32-bit slabs; sixteen loads are in flight at a time, only the additions are a chain)
// MULTI false: the kernel was launched for a single tensor and carries none of the code for parts.
template <bool MULTI>
__device__ __forceinline__ float la_in(const void* p, int dtype, int parts, size_t stride, size_t i) {
    if (!MULTI || parts == 1) return la_any(p, dtype, i);
    const float* f = reinterpret_cast<const float*>(p) + i;
    float v = 0.f;
    for (int s0 = 0; s0 < parts; s0 += 16) {
        float part[16];
#pragma unroll
        for (int u = 0; u < 16; ++u) part[u] = s0 + u < parts ? f[(size_t)(s0 + u) * stride] : 0.f;
#pragma unroll
        for (int u = 0; u < 16; ++u)
            if (s0 + u < parts) v = (s0 + u == 0) ? part[u] : v + part[u];
    }
    return v;
}

// ---------------------------------------------------------------------------------------------------
// prepare: grid (tiles of TT tokens, heads), 128 threads
// ---------------------------------------------------------------------------------------------------
constexpr int PREP_RK = 32;      // columns of the low-rank map taken at a time

// TT tokens a CTA: the head's slab of the low-rank matrix is read once for all of them (prompts: 8); a step of few
// tokens takes one token a CTA, so that tokens x heads CTAs share the work.
template <int TT, bool MULTI>
__global__ void __launch_bounds__(128)
linattn_prepare_kernel(const void* __restrict__ fused, int in_dtype, int row_stride, int parts, size_t part_stride,
                       int q_off, int k_off, int v_off, int a_off, int n, int H, int D, int V, int rank,
                       const int* __restrict__ positions, const float* __restrict__ inv_freq, int rot_dim,
                       float q_scale, float k_scale, const void* __restrict__ w2, const void* __restrict__ b2,
                       int w_dtype, float inv_tau, float* __restrict__ q, float* __restrict__ k,
                       float* __restrict__ v, float* __restrict__ decay) {
    __shared__ __align__(16) float low_s[PREP_RK][TT];      // the tokens' low-rank vectors, a run of PREP_RK columns at a time
    pdl_begin();
    const int t_lo = blockIdx.x * TT, h = blockIdx.y;
    const int count = min(TT, n - t_lo);
    const int half = rot_dim >> 1, rest = D - rot_dim;
    // q and k: the rotated pairs, then the channels behind them; v: a copy.  One flat loop each over (token, element),
    // so that a thread's loads do not wait for one another.
    for (int which = 0; which < 2; ++which) {
        const int off = (which ? k_off : q_off) + h * D;
        float* base = which ? k : q;
        const float scale = which ? k_scale : q_scale;
        for (int idx = threadIdx.x; idx < count * half; idx += blockDim.x) {
            const int tt = idx / half, j = idx - tt * half, t = t_lo + tt;
            const size_t row = (size_t)t * row_stride + off;
            float sn, cs, y1, y2;
            sincosf((float)positions[t] * inv_freq[j], &sn, &cs);
            rotate_pair(la_in<MULTI>(fused, in_dtype, parts, part_stride, row + j),
                        la_in<MULTI>(fused, in_dtype, parts, part_stride, row + j + half), sn, cs, y1, y2);
            float* dst = base + ((size_t)t * H + h) * D;
            dst[j] = y1 * scale;
            dst[j + half] = y2 * scale;
        }
        for (int idx = threadIdx.x; idx < count * rest; idx += blockDim.x) {
            const int tt = idx / rest, c = rot_dim + idx - tt * rest, t = t_lo + tt;
            base[((size_t)t * H + h) * D + c] = la_in<MULTI>(fused, in_dtype, parts, part_stride, (size_t)t * row_stride + off + c) * scale;
        }
    }
    for (int idx = threadIdx.x; idx < count * V; idx += blockDim.x) {
        const int tt = idx / V, c = idx - tt * V, t = t_lo + tt;
        v[((size_t)t * H + h) * V + c] = la_in<MULTI>(fused, in_dtype, parts, part_stride, (size_t)t * row_stride + v_off + h * V + c);
    }
    if (a_off < 0) return;
    // z[token][channel] = b2[channel] + sum_r low[token][r] * w2[channel][r]: a thread a channel, TT sums each; the
    // thread takes PREP_RK of its channel's weights into registers at a time (16-byte loads where the rows allow), the
    // tokens' low-rank vectors come from shared memory.  The sum over r runs in ascending order whatever the tiling.
    const bool vec = ((uintptr_t)w2 & 15) == 0 && rank % 8 == 0;
    for (int c0 = 0; c0 < D; c0 += 128) {
        const int c = c0 + threadIdx.x;
        const size_t ch = (size_t)h * D + min(c, D - 1);
        float z[TT];
        const float bias = la_any(b2, w_dtype, ch);
#pragma unroll
        for (int tt = 0; tt < TT; ++tt) z[tt] = bias;
        for (int r0 = 0; r0 < rank; r0 += PREP_RK) {
            const int rk = min(PREP_RK, rank - r0);
            __syncthreads();
            for (int idx = threadIdx.x; idx < TT * PREP_RK; idx += blockDim.x) {
                const int r = idx / TT, tt = idx % TT;
                low_s[r][tt] = (tt < count && r < rk)
                    ? la_in<MULTI>(fused, in_dtype, parts, part_stride, (size_t)(t_lo + tt) * row_stride + a_off + r0 + r) : 0.f;
            }
            float wr[PREP_RK];
            if (vec && rk == PREP_RK) {
                if (w_dtype == WLLM_BF16) {
                    const uint4* src = reinterpret_cast<const uint4*>(reinterpret_cast<const bf16*>(w2) + ch * rank + r0);
                    uint4 raw[PREP_RK / 8];
#pragma unroll
                    for (int u = 0; u < PREP_RK / 8; ++u) raw[u] = src[u];
#pragma unroll
                    for (int u = 0; u < PREP_RK / 8; ++u) {
                        const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw[u]);
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const float2 f = __bfloat1622float2(h2[e]);
                            wr[u * 8 + 2 * e] = f.x;
                            wr[u * 8 + 2 * e + 1] = f.y;
                        }
                    }
                } else {
                    const float4* src = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(w2) + ch * rank + r0);
#pragma unroll
                    for (int u = 0; u < PREP_RK / 4; ++u) {
                        const float4 f = src[u];
                        wr[u * 4] = f.x; wr[u * 4 + 1] = f.y; wr[u * 4 + 2] = f.z; wr[u * 4 + 3] = f.w;
                    }
                }
            } else {
#pragma unroll
                for (int r = 0; r < PREP_RK; ++r) wr[r] = r < rk ? la_any(w2, w_dtype, ch * rank + r0 + r) : 0.f;
            }
            __syncthreads();
#pragma unroll
            for (int r = 0; r < PREP_RK; ++r) {
#pragma unroll
                for (int tt = 0; tt < TT; ++tt) z[tt] = fmaf(low_s[r][tt], wr[r], z[tt]);
            }
        }
        if (c < D) {
#pragma unroll
            for (int tt = 0; tt < TT; ++tt) {
                if (tt >= count) break;
                // log(sigmoid(z)) = min(z, 0) - log(1 + e^-|z|), exact at both ends
                const float log_sig = fminf(z[tt], 0.f) - log1pf(expf(-fabsf(z[tt])));
                decay[((size_t)(t_lo + tt) * H + h) * D + c] = expf(log_sig * inv_tau);
            }
        }
    }
}

WLLM_API int wllm_linattn_prepare(const void* fused, int in_dtype, int row_stride, int parts, long long part_stride, int q_off,
                                  int k_off, int v_off, int a_off, int n, int H, int D, int V, int rank, const int* positions,
                                  const float* inv_freq, int rot_dim, float q_scale, float k_scale, const void* w2,
                                  const void* b2, int w_dtype, float tau, float* q, float* k, float* v, float* decay,
                                  cudaStream_t stream) {
    if (n <= 0) return WLLM_OK;
    if (H <= 0 || H > 65535 || D <= 0 || V <= 0 || parts < 1 || rot_dim < 0 || rot_dim > D || (rot_dim & 1)) return WLLM_BAD_SIZE;
    if (a_off >= 0 && (rank <= 0 || !(tau > 0.f) || !w2 || !b2 || !decay)) return WLLM_BAD_SIZE;
    if ((in_dtype != WLLM_BF16 && in_dtype != WLLM_F32) || (a_off >= 0 && w_dtype != WLLM_BF16 && w_dtype != WLLM_F32))
        return WLLM_BAD_DTYPE;
#define PREP2(TT, M) wllm_launch(linattn_prepare_kernel<TT, M>, dim3((n + TT - 1) / TT, H), 128, 0, stream, fused, \
        in_dtype, row_stride, parts, (size_t)part_stride, q_off, k_off, v_off, a_off, n, H, D, V, rank, positions, \
        inv_freq, rot_dim, q_scale, k_scale, w2, b2, w_dtype, a_off >= 0 ? 1.0f / tau : 0.f, q, k, v, decay)
#define PREP(TT) (parts > 1 ? PREP2(TT, true) : PREP2(TT, false))
    if ((long long)n * H >= 2048) return PREP(8);
    return PREP(1);
#undef PREP
#undef PREP2
}

// ---------------------------------------------------------------------------------------------------
// scan
// ---------------------------------------------------------------------------------------------------
constexpr int LA_CPT = 16;       // key channels a thread holds of each of its columns of S (a multiple of 4)
constexpr int LA_TT = 8;         // tokens of a tile
constexpr int LA_COLS = 64;      // value columns of a CTA: two a lane (lane and lane + 32)

__device__ __forceinline__ void la_cp4(float* smem_dst, const float* src) {
    const unsigned dst = (unsigned)__cvta_generic_to_shared(smem_dst);
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void la_cp16(float* smem_dst, const float* src) {      // both 16-byte aligned
    const unsigned dst = (unsigned)__cvta_generic_to_shared(smem_dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}

// MODE 0  a request's tokens of the step in one walk: from its state slot, outputs written, back to the slot.
// Long portions are cut into segments of `seg_len` tokens that are walked at the same time (grid z = request * max_seg + segment):
// MODE 1  every segment but a request's last, from a zero state and without outputs: its local end state L and the
//         product A of its decays per key channel go to scratch[(request * max_seg + segment + 1)] (the place of the
//         next segment's start).  linattn_combine_kernel then turns them into start states in segment order:
//         start_(j+1) = diag(A_j) start_j + L_j, start_0 = the slot's state (copied beside them).
// MODE 2  every segment again, from its start state, with outputs; the last one leaves the request's new state.
// The state that a token meets is the same up to rounding in all modes; the arithmetic from there is the same.
//
// A warp holds a run of `cpt` key channels (a multiple of 4, at most 16) of 64 columns of S: a lane two columns, in
// registers.  A token's q, k and decay are the same for all lanes: they are read from shared memory four channels at
// a time, and with two columns a lane every such read feeds eight multiply-adds; one column a lane and one channel
// a read left the kernel waiting for shared memory (a read a multiply-add).
// FULL: every warp holds LA_CPT channels (the head's key size is a multiple of 16): the loops carry no guards.
template <bool PER_CHANNEL, int MODE, bool FULL>
__global__ void __launch_bounds__(512)
linattn_scan_kernel(const float* __restrict__ q, const float* __restrict__ k, const float* __restrict__ v,
                    const float* __restrict__ decay, const float* __restrict__ head_decay, float* __restrict__ state,
                    float* __restrict__ out, const int* __restrict__ req_q_start, const int* __restrict__ req_q_len,
                    const int* __restrict__ req_slot, int H, int D, int V, int cpt, int seg_len, int max_seg,
                    float* __restrict__ seg_state, float* __restrict__ seg_decay) {
    extern __shared__ __align__(16) float la_smem[];
    pdl_begin();
    const int r = MODE == 0 ? blockIdx.z : blockIdx.z / max_seg, seg = MODE == 0 ? 0 : blockIdx.z % max_seg, h = blockIdx.y;
    const int req_len = req_q_len[r], slot = req_slot[r];
    if (req_len <= 0 || slot < 0) return;                     // a request that brings no token
    const int nseg = MODE == 0 ? 1 : (req_len + seg_len - 1) / seg_len;
    if (seg >= nseg || (MODE == 1 && seg == nseg - 1)) return;
    const int tok_lo = MODE == 0 ? 0 : seg * seg_len;
    const int q_len = MODE == 0 ? req_len : min(req_len - tok_lo, seg_len);      // tokens of this walk
    const int t0 = req_q_start[r] + tok_lo;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
    const int j0 = blockIdx.x * LA_COLS + lane, j1 = j0 + 32;  // this lane's columns of S
    const bool col0 = j0 < V, col1 = j1 < V;
    const int c_lo = warp * cpt, c_hi = min(D, c_lo + cpt);   // this warp's key channels
    // shared memory: two stages of [q | k | (a) | v] for LA_TT tokens (each run of D padded to a multiple of 4), then
    // two rounds of the warps' partial sums
    const int Dp = (D + 3) & ~3, NA = PER_CHANNEL ? 3 : 2;
    const int per_token = NA * Dp + LA_COLS;
    float* stage0 = la_smem;
    float* red = la_smem + 2 * LA_TT * per_token;             // [2][warps][LA_TT][64]

    float S0[LA_CPT], S1[LA_CPT], P[LA_CPT];
    float* Sg = state + (((size_t)slot * H + h) * D) * V;
    // (a request of several segments reads every start from the scratch, the first one too: its last segment
    // may write the slot before its first one has started)
    const float* St = (MODE == 2 && nseg > 1) ? seg_state + (((size_t)(r * max_seg + seg) * H + h) * D) * V : Sg;
#pragma unroll
    for (int i = 0; i < LA_CPT; ++i) {
        const bool ch = MODE != 1 && (FULL || c_lo + i < c_hi);
        S0[i] = (ch && col0) ? St[(size_t)(c_lo + i) * V + j0] : 0.f;
        S1[i] = (ch && col1) ? St[(size_t)(c_lo + i) * V + j1] : 0.f;
        P[i] = 1.f;
    }
    const float fixed = PER_CHANNEL ? 0.f : head_decay[h];

    // rows of whole 16-byte pieces (key sizes in steps of 16, value sizes in steps of 4, aligned buffers): a warp a token,
    // a lane a piece of q, k and the decay, sixteen lanes a piece of v; no division, a quarter of the copies
    const bool pieces = FULL && (V & 3) == 0 &&
        ((((uintptr_t)q | (uintptr_t)k | (uintptr_t)v | (PER_CHANNEL ? (uintptr_t)decay : 0)) & 15) == 0);
    auto load_tile = [&](int tile, int stage) {
        float* dst = stage0 + (size_t)stage * LA_TT * per_token;
        const int first = t0 + tile * LA_TT, count = min(LA_TT, q_len - tile * LA_TT);
        if (pieces) {
            for (int tt = warp; tt < count; tt += warps) {
                const size_t at = ((size_t)(first + tt) * H + h) * D;
                float* d = dst + tt * per_token;
                for (int c = 4 * lane; c < D; c += 128) {
                    la_cp16(d + c, q + at + c);
                    la_cp16(d + Dp + c, k + at + c);
                    if (PER_CHANNEL) la_cp16(d + 2 * Dp + c, decay + at + c);
                }
                if (lane < LA_COLS / 4) {
                    const int cc = blockIdx.x * LA_COLS + 4 * lane;
                    const float* vrow = v + ((size_t)(first + tt) * H + h) * V;
                    if (cc + 3 < V) la_cp16(d + NA * Dp + 4 * lane, vrow + cc);
                    else
                        for (int e = 0; e < 4; ++e) la_cp4(d + NA * Dp + 4 * lane + e, vrow + min(cc + e, V - 1));
                }
            }
            asm volatile("cp.async.commit_group;" ::: "memory");
            return;
        }
        for (int idx = threadIdx.x; idx < count * D; idx += blockDim.x) {
            const int tt = idx / D, c = idx - tt * D;
            const size_t at = ((size_t)(first + tt) * H + h) * D + c;
            float* d = dst + tt * per_token + c;
            la_cp4(d, q + at);
            la_cp4(d + Dp, k + at);
            if (PER_CHANNEL) la_cp4(d + 2 * Dp, decay + at);
        }
        for (int idx = threadIdx.x; idx < count * LA_COLS; idx += blockDim.x) {
            const int tt = idx / LA_COLS, cc = idx % LA_COLS;
            la_cp4(dst + tt * per_token + NA * Dp + cc,
                   v + ((size_t)(first + tt) * H + h) * V + min(blockIdx.x * LA_COLS + cc, V - 1));
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };

    const int tiles = (q_len + LA_TT - 1) / LA_TT;
    load_tile(0, 0);
    int round = 0;
    for (int tile = 0; tile < tiles; ++tile) {
        const int stage = tile & 1;
        if (tile + 1 < tiles) {
            load_tile(tile + 1, stage ^ 1);
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncthreads();
        const float* base = stage0 + (size_t)stage * LA_TT * per_token;
        const int count = min(LA_TT, q_len - tile * LA_TT);
        float p0[LA_TT], p1[LA_TT];          // this warp's share of the tile's outputs, two columns
#pragma unroll
        for (int tt = 0; tt < LA_TT; ++tt) {
            p0[tt] = p1[tt] = 0.f;
            if (tt < count) {
                const float* qs = base + tt * per_token;
                const float v0 = qs[NA * Dp + lane], v1 = qs[NA * Dp + 32 + lane];
#pragma unroll
                for (int i4 = 0; i4 < LA_CPT; i4 += 4) {
                    if (FULL || c_lo + i4 < c_hi) {
                        const float4 q4 = *reinterpret_cast<const float4*>(qs + c_lo + i4);
                        const float4 k4 = *reinterpret_cast<const float4*>(qs + Dp + c_lo + i4);
                        float4 a4 = make_float4(fixed, fixed, fixed, fixed);
                        if (PER_CHANNEL) a4 = *reinterpret_cast<const float4*>(qs + 2 * Dp + c_lo + i4);
                        const float qe[4] = {q4.x, q4.y, q4.z, q4.w}, ke[4] = {k4.x, k4.y, k4.z, k4.w}, ae[4] = {a4.x, a4.y, a4.z, a4.w};
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            if (FULL || c_lo + i4 + e < c_hi) {   // (the last channels of a head whose size is no multiple of 4)
                                S0[i4 + e] = fmaf(ae[e], S0[i4 + e], ke[e] * v0);
                                S1[i4 + e] = fmaf(ae[e], S1[i4 + e], ke[e] * v1);
                                if (MODE == 1) P[i4 + e] *= ae[e];
                                else {
                                    p0[tt] = fmaf(S0[i4 + e], qe[e], p0[tt]);
                                    p1[tt] = fmaf(S1[i4 + e], qe[e], p1[tt]);
                                }
                            }
                        }
                    }
                }
            }
        }
        if (MODE == 1) {
            __syncthreads();       // the stage is read to its end before the tile after next lands in it
            continue;
        }
        // the warps' sums meet once a tile: red[round][warp][token][64]; then warp w adds up the tokens w, w + warps, ..
        // in warp order (the sum of a token depends on nothing but the token)
        float* mine = red + ((size_t)(round * warps + warp) * LA_TT) * 64;
#pragma unroll
        for (int tt = 0; tt < LA_TT; ++tt) {
            mine[tt * 64 + lane] = p0[tt];
            mine[tt * 64 + 32 + lane] = p1[tt];
        }
        __syncthreads();           // (also: every warp has read the stage to its end)
        for (int tt = warp; tt < count; tt += warps) {
            const float* from = red + ((size_t)(round * warps) * LA_TT + tt) * 64 + lane;
            float o0 = from[0], o1 = from[32];
            for (int w = 1; w < warps; ++w) {
                o0 += from[(size_t)w * LA_TT * 64];
                o1 += from[(size_t)w * LA_TT * 64 + 32];
            }
            float* orow = out + ((size_t)(t0 + tile * LA_TT + tt) * H + h) * V;
            if (col0) orow[j0] = o0;
            if (col1) orow[j1] = o1;
        }
        round ^= 1;
    }
    if (MODE == 1) {
        float* Ld = seg_state + (((size_t)(r * max_seg + seg + 1) * H + h) * D) * V;
        float* Ad = seg_decay + ((size_t)(r * max_seg + seg + 1) * H + h) * D;
#pragma unroll
        for (int i = 0; i < LA_CPT; ++i)
            if (FULL || c_lo + i < c_hi) {
                if (col0) Ld[(size_t)(c_lo + i) * V + j0] = S0[i];
                if (col1) Ld[(size_t)(c_lo + i) * V + j1] = S1[i];
                if (blockIdx.x == 0 && lane == 0) Ad[c_lo + i] = P[i];
            }
        return;
    }
    if (MODE == 0 || seg == nseg - 1) {
#pragma unroll
        for (int i = 0; i < LA_CPT; ++i)
            if (FULL || c_lo + i < c_hi) {
                if (col0) Sg[(size_t)(c_lo + i) * V + j0] = S0[i];
                if (col1) Sg[(size_t)(c_lo + i) * V + j1] = S1[i];
            }
    }
}

// start states of the segments 1 .. nseg-1 of every request, in place of their local end states; grid (D*V / 256, H, requests)
__global__ void linattn_combine_kernel(const float* __restrict__ state, const int* __restrict__ req_q_len,
                                       const int* __restrict__ req_slot, int H, int D, int V, int seg_len, int max_seg,
                                       float* __restrict__ seg_state, const float* __restrict__ seg_decay) {
    pdl_begin();
    const int r = blockIdx.z, h = blockIdx.y;
    const int req_len = req_q_len[r], slot = req_slot[r];
    if (req_len <= 0 || slot < 0) return;
    const int nseg = (req_len + seg_len - 1) / seg_len;
    const int e = blockIdx.x * blockDim.x + threadIdx.x;
    if (nseg <= 1 || e >= D * V) return;
    const int d = e / V;
    float cur = state[(((size_t)slot * H + h) * D) * V + e];
    seg_state[((size_t)(r * max_seg) * H + h) * D * V + e] = cur;
    for (int sgm = 1; sgm < nseg; ++sgm) {
        const size_t at = (size_t)(r * max_seg + sgm) * H + h;
        cur = fmaf(seg_decay[at * D + d], cur, seg_state[at * D * V + e]);
        seg_state[at * D * V + e] = cur;
    }
}

// q, k: [n, H, D]; v, out: [n, H, V]; decay: [n, H, D] per key channel, or null with head_decay [H];
// state: [slots, H, D, V].  Requests by start, length and state slot; a length of 0 or a slot of -1 is passed by.
// seg_len > 0: portions longer than that are cut into segments that run side by side (at most max_seg a request, which
// must cover the longest portion); seg_state holds requests * max_seg * H * D * V floats, seg_decay requests * max_seg * H * D.
WLLM_API int wllm_linattn_scan(const float* q, const float* k, const float* v, const float* decay, const float* head_decay,
                               float* state, float* out, const int* req_q_start, const int* req_q_len, const int* req_slot,
                               int requests, int H, int D, int V, int seg_len, int max_seg, float* seg_state, float* seg_decay,
                               cudaStream_t stream) {
    if (requests <= 0) return WLLM_OK;
    if (H <= 0 || H > 65535 || requests > 65535 || D <= 0 || D > 16 * LA_CPT || V <= 0) return WLLM_BAD_SIZE;
    if (!decay && !head_decay) return WLLM_BAD_SIZE;
    const bool cut = seg_len > 0 && max_seg > 1;
    if (cut && (!seg_state || !seg_decay || (long long)requests * max_seg > 65535)) return WLLM_BAD_SIZE;
    const int most = (D + LA_CPT - 1) / LA_CPT;
    const int cpt = (((D + most - 1) / most) + 3) & ~3;          // a multiple of 4, at most LA_CPT
    const int warps = (D + cpt - 1) / cpt;
    const int vtiles = (V + LA_COLS - 1) / LA_COLS;
    const size_t smem = ((size_t)2 * LA_TT * ((decay ? 3 : 2) * ((D + 3) & ~3) + LA_COLS) + 2 * warps * LA_TT * 64) * sizeof(float);
    const bool full = cpt == LA_CPT && D % LA_CPT == 0;
    static bool raised = false;
    if (!raised) {
        cudaError_t e = cudaSuccess;
#define RAISE(PC, M) if (e == cudaSuccess) e = cudaFuncSetAttribute(linattn_scan_kernel<PC, M, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024); \
        if (e == cudaSuccess) e = cudaFuncSetAttribute(linattn_scan_kernel<PC, M, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024)
        RAISE(true, 0); RAISE(true, 1); RAISE(true, 2); RAISE(false, 0); RAISE(false, 1); RAISE(false, 2);
#undef RAISE
        if (e != cudaSuccess) return 1000 + (int)e;
        raised = true;
    }
#define SCAN2(PC, MODE, F, GRID) wllm_launch(linattn_scan_kernel<PC, MODE, F>, GRID, warps * 32, smem, stream, q, k, v, decay, head_decay, \
        state, out, req_q_start, req_q_len, req_slot, H, D, V, cpt, seg_len, max_seg, seg_state, seg_decay)
#define SCAN(PC, MODE, GRID) (full ? SCAN2(PC, MODE, true, GRID) : SCAN2(PC, MODE, false, GRID))
    if (!cut) {
        const dim3 grid(vtiles, H, requests);
        return decay ? SCAN(true, 0, grid) : SCAN(false, 0, grid);
    }
    const dim3 grid(vtiles, H, requests * max_seg);
    int st = decay ? SCAN(true, 1, grid) : SCAN(false, 1, grid);
    if (st != WLLM_OK) return st;
    st = wllm_launch(linattn_combine_kernel, dim3((D * V + 255) / 256, H, requests), 256, 0, stream, (const float*)state,
                     req_q_len, req_slot, H, D, V, seg_len, max_seg, seg_state, (const float*)seg_decay);
    if (st != WLLM_OK) return st;
    return decay ? SCAN(true, 2, grid) : SCAN(false, 2, grid);
#undef SCAN
#undef SCAN2
}

// ---------------------------------------------------------------------------------------------------
// head norm and gate: grid (tokens, heads), one warp
// ---------------------------------------------------------------------------------------------------
template <typename TO, bool MULTI>
__global__ void head_gate_norm_kernel(const float* __restrict__ o, const void* __restrict__ fused, int in_dtype, int row_stride,
                                      int parts, size_t part_stride, int g_off, const void* __restrict__ w, int w_dtype,
                                      float eps, TO* __restrict__ out, int H, int V) {
    pdl_begin();
    const int t = blockIdx.x, h = blockIdx.y, lane = threadIdx.x;
    const float* orow = o + ((size_t)t * H + h) * V;
    float ss = 0.f;
    for (int c = lane; c < V; c += 32) ss = fmaf(orow[c], orow[c], ss);
    ss = warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss / (float)V + eps);
    const size_t grow = (size_t)t * row_stride + g_off + (size_t)h * V;
    for (int c = lane; c < V; c += 32) {
        const float g = la_in<MULTI>(fused, in_dtype, parts, part_stride, grow + c);
        float y = orow[c] * inv;
        if (w) y *= la_any(w, w_dtype, c);
        out[((size_t)t * H + h) * V + c] = from_f32<TO>(y * (g / (1.0f + expf(-g))));
    }
}

// out[n, H*V] = o / sqrt(mean_V(o^2) + eps) * w[V] (w may be null) * silu(g), g = fused[:, g_off + h*V + c]
WLLM_API int wllm_head_gate_norm(const float* o, const void* fused, int in_dtype, int row_stride, int parts,
                                 long long part_stride, int g_off, const void* w, int w_dtype, float eps, void* out,
                                 int out_dtype, int n, int H, int V, cudaStream_t stream) {
    if (n <= 0) return WLLM_OK;
    if (H <= 0 || H > 65535 || V <= 0 || parts < 1) return WLLM_BAD_SIZE;
    if ((in_dtype != WLLM_BF16 && in_dtype != WLLM_F32) || (w && w_dtype != WLLM_BF16 && w_dtype != WLLM_F32)) return WLLM_BAD_DTYPE;
#define GATE(TO, M) wllm_launch(head_gate_norm_kernel<TO, M>, dim3(n, H), 32, 0, stream, o, fused, in_dtype, row_stride, parts, \
        (size_t)part_stride, g_off, w, w_dtype, eps, (TO*)out, H, V)
    if (out_dtype == WLLM_BF16) return parts > 1 ? GATE(bf16, true) : GATE(bf16, false);
    if (out_dtype == WLLM_F32) return parts > 1 ? GATE(float, true) : GATE(float, false);
#undef GATE
    return WLLM_BAD_DTYPE;
}
