// Routed experts: every token runs `top` of E small gated feed-forward units, chosen by a router.
//
//   route    z = W_router h in 32-bit (W_router is held in 32-bit; h as the norm left it), s = softmax(z) over all
//            experts.  The experts form `groups` equal groups of neighbours; a group's score is its best expert's, and
//            only experts of the `groups_kept` best groups can be chosen.  The `top` best of those are the token's
//            experts, in descending order of score (ties: the lower index first), weighted by their scores as they
//            are.  A shared unit's gate, sigmoid(w_gate . h), is worked out along the way.  One CTA a token; every
//            dot product is a lane's strided chain and the warp's tree, so a token's choice and weights do not depend
//            on the batch.
//   plan     the (token, rank) pairs sorted by expert, stably: count[e], offset[e], sorted[r] = pair, place[pair] = r.
//            A warp an expert, by ballots over the pair list; no atomics, so the order is the same every time.
//   experts  grouped products over the sorted rows: act = unit(gate_e a, up_e a) for the rows of expert e (a gathered
//            from the tokens' rows), then y = down_e act, 32-bit accumulation, each output one ascending chain over k.
//            A CTA takes a tile of rows of ONE expert and a tile of columns; the grid is sized from the pair count
//            and E alone (tiles that find no rows leave at once), so a captured step can replay it.
//   combine  out[token] = sum over the token's ranks, in rank order, of weight * y[place] (+ gate * shared unit).
//
// The gated unit is the clamped one: g = min(gate, limit), u = clamp(up, -limit, limit), g sigmoid(slope g) (u + 1).
#include "common.cuh"

constexpr int MOE_MAX_EXPERTS = 1024;

template <typename T>
__global__ void __launch_bounds__(128)
moe_route_kernel(const T* __restrict__ h, const float* __restrict__ w_router, const float* __restrict__ w_gate,
                 int* __restrict__ chosen, float* __restrict__ weights, float* __restrict__ gate_out, int H, int E, int top,
                 int groups, int groups_kept) {
    extern __shared__ float route_smem[];          // [H] the token's row, [E] scores, [groups] group scores
    float* hs = route_smem;
    float* sc = hs + H;
    float* gs = sc + E;
    pdl_begin();
    const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
    for (int c = threadIdx.x; c < H; c += blockDim.x) hs[c] = to_f32(h[(size_t)t * H + c]);
    __syncthreads();
    for (int e = warp; e < E + (w_gate != nullptr ? 1 : 0); e += nwarps) {
        const float* w = e < E ? w_router + (size_t)e * H : w_gate;
        float acc = 0.f;
        for (int c = lane; c < H; c += 32) acc = fmaf(w[c], hs[c], acc);
        acc = warp_sum(acc);
        if (lane == 0) {
            if (e < E) sc[e] = acc; else gate_out[t] = 1.0f / (1.0f + expf(-acc));
        }
    }
    __syncthreads();
    if (warp == 0) {
        float m = -INFINITY;
        for (int e = lane; e < E; e += 32) m = fmaxf(m, sc[e]);
        m = warp_max(m);
        float sum = 0.f;
        for (int e = lane; e < E; e += 32) { const float p = expf(sc[e] - m); sc[e] = p; sum += p; }
        sum = warp_sum(sum);
        const float inv = 1.0f / sum;
        for (int e = lane; e < E; e += 32) sc[e] *= inv;
        __syncwarp();
        const int per = E / groups;
        for (int g = lane; g < groups; g += 32) {
            float best = -INFINITY;
            for (int j = 0; j < per; ++j) best = fmaxf(best, sc[g * per + j]);
            gs[g] = best;
        }
        __syncwarp();
        // the groups that stay: groups_kept times the best one left (ties: the lower index); the others' experts leave
        if (groups_kept < groups) {
            for (int round = 0; round < groups_kept; ++round) {
                float best = -INFINITY; int at = 0x7fffffff;
                for (int g = lane; g < groups; g += 32) { const float v = gs[g]; if (v > best) { best = v; at = g; } }
                for (int o = 16; o > 0; o >>= 1) {
                    const float ob = __shfl_xor_sync(0xffffffffu, best, o); const int oa = __shfl_xor_sync(0xffffffffu, at, o);
                    if (ob > best || (ob == best && oa < at)) { best = ob; at = oa; }
                }
                if (lane == 0) gs[at] = -2.0f;              // marked as kept (scores lie in [0, 1])
                __syncwarp();
            }
            for (int e = lane; e < E; e += 32) if (gs[e / per] != -2.0f) sc[e] = -1.0f;
            __syncwarp();
        }
        for (int k = 0; k < top; ++k) {
            float best = -INFINITY; int at = 0x7fffffff;
            for (int e = lane; e < E; e += 32) { const float v = sc[e]; if (v > best) { best = v; at = e; } }
            for (int o = 16; o > 0; o >>= 1) {
                const float ob = __shfl_xor_sync(0xffffffffu, best, o); const int oa = __shfl_xor_sync(0xffffffffu, at, o);
                if (ob > best || (ob == best && oa < at)) { best = ob; at = oa; }
            }
            if (lane == 0) { chosen[(size_t)t * top + k] = at; weights[(size_t)t * top + k] = best; sc[at] = -3.0f; }
            __syncwarp();
        }
    }
}

// grid: E warps (4 a CTA).  count[e] = pairs whose expert is e.
__global__ void __launch_bounds__(128) moe_count_kernel(const int* __restrict__ chosen, int pairs, int E, int* __restrict__ count) {
    pdl_begin();
    const int e = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (e >= E) return;
    int c = 0;
    for (int p0 = 0; p0 < pairs; p0 += 32) {
        const int p = p0 + lane;
        c += __popc(__ballot_sync(0xffffffffu, p < pairs && chosen[p] == e));
    }
    if (lane == 0) count[e] = c;
}

// offset[e] = count[0] + .. + count[e-1] (offset[E] = pairs); the pairs of expert e in ascending order fill the sorted
// rows from offset[e]: sorted[r] = pair, place[pair] = r.
__global__ void __launch_bounds__(128) moe_place_kernel(const int* __restrict__ chosen, int pairs, int E, const int* __restrict__ count,
                                                        int* __restrict__ offset, int* __restrict__ sorted, int* __restrict__ place) {
    pdl_begin();
    const int e = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (e >= E) return;
    int before = 0;
    for (int j = lane; j < e; j += 32) before += count[j];
    for (int o = 16; o > 0; o >>= 1) before += __shfl_xor_sync(0xffffffffu, before, o);
    if (lane == 0) {
        offset[e] = before;
        if (e == E - 1) offset[E] = before + count[e];
    }
    int at = before;
    for (int p0 = 0; p0 < pairs; p0 += 32) {
        const int p = p0 + lane;
        const bool mine = p < pairs && chosen[p] == e;
        const unsigned b = __ballot_sync(0xffffffffu, mine);
        if (mine) {
            const int r = at + __popc(b & ((1u << lane) - 1u));
            sorted[r] = p;
            place[p] = r;
        }
        at += __popc(b);
    }
}

constexpr int GM = 32, GN = 64, GK = 16;

// One tile of rows (of one expert) by one tile of columns.  GATED: w holds [E][2 N][K] (gate rows, then up rows), the
// rows of a are gathered (token = sorted[r] / top) and out[r][c] = unit(gate, up) in TO; else w is [E][N][K], the rows
// of a are the sorted rows and out is 32-bit.  Thread (ty, tx) of 16 x 16 owns rows ty, ty + 16 and columns tx + 16 j.
template <typename T, typename TO, bool GATED>
__global__ void __launch_bounds__(256)
moe_grouped_kernel(const T* __restrict__ a, int a_stride, const T* __restrict__ w, TO* __restrict__ out, int N, int K,
                   const int* __restrict__ offset, const int* __restrict__ sorted, int E, int top, float limit, float slope) {
    __shared__ float As[GK][GM + 1];
    __shared__ float Ws[GATED ? 2 : 1][GK][GN + 1];
    __shared__ int s_expert, s_row0, s_rows;
    pdl_begin();
    if (threadIdx.x == 0) {
        // the tile's expert: tiles are dealt expert by expert, ceil(count / GM) each
        int tile = blockIdx.y, e = 0, found = -1, row0 = 0, rows = 0;
        for (; e < E; ++e) {
            const int lo = offset[e], cnt = offset[e + 1] - lo, tiles = (cnt + GM - 1) / GM;
            if (tile < tiles) { found = e; row0 = lo + tile * GM; rows = min(GM, cnt - tile * GM); break; }
            tile -= tiles;
        }
        s_expert = found; s_row0 = row0; s_rows = rows;
    }
    __syncthreads();
    const int e = s_expert;
    if (e < 0) return;
    const int row0 = s_row0, rows = s_rows, col0 = blockIdx.x * GN;
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    const T* we = w + (size_t)e * (GATED ? 2 : 1) * N * K;
    float acc[GATED ? 2 : 1][2][4];
#pragma unroll
    for (int g = 0; g < (GATED ? 2 : 1); ++g)
#pragma unroll
        for (int i = 0; i < 2; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) acc[g][i][j] = 0.f;
    // which row of `a` each of the tile's rows reads
    const int lr = threadIdx.x >> 3;                 // 0..31: the row this thread loads (two k each)
    int src_row = -1;
    if (lr < rows) src_row = GATED ? sorted[row0 + lr] / top : row0 + lr;
    for (int k0 = 0; k0 < K; k0 += GK) {
        {
            const int kk = (threadIdx.x & 7) * 2;
#pragma unroll
            for (int u = 0; u < 2; ++u) {
                const int k = k0 + kk + u;
                As[kk + u][lr] = (src_row >= 0 && k < K) ? to_f32(a[(size_t)src_row * a_stride + k]) : 0.f;
            }
        }
#pragma unroll
        for (int g = 0; g < (GATED ? 2 : 1); ++g) {
            for (int idx = threadIdx.x; idx < GN * GK; idx += 256) {
                const int c = idx / GK, kk = idx % GK, col = col0 + c, k = k0 + kk;
                Ws[g][kk][c] = (col < N && k < K) ? to_f32(we[((size_t)g * N + col) * K + k]) : 0.f;
            }
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < GK; ++kk) {
            const float a0 = As[kk][ty], a1 = As[kk][ty + 16];
#pragma unroll
            for (int g = 0; g < (GATED ? 2 : 1); ++g)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float wv = Ws[g][kk][tx + 16 * j];
                    acc[g][0][j] = fmaf(a0, wv, acc[g][0][j]);
                    acc[g][1][j] = fmaf(a1, wv, acc[g][1][j]);
                }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int r = ty + 16 * i;
        if (r >= rows) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int col = col0 + tx + 16 * j;
            if (col >= N) continue;
            float v = acc[0][i][j];
            if (GATED) {
                const float g = fminf(v, limit), u = fminf(fmaxf(acc[GATED ? 1 : 0][i][j], -limit), limit);
                v = (g / (1.0f + expf(-slope * g))) * (u + 1.0f);
            }
            out[(size_t)(row0 + r) * N + col] = from_f32<TO>(v);
        }
    }
}

// out[t][c] = sum_k weights[t][k] * y[place[t top + k]][c]  (+ gate[t] * shared[t][c], shared a tensor of TS or `parts`
// 32-bit partial sums added in order first)
template <typename TS>
__global__ void __launch_bounds__(256)
moe_combine_kernel(const float* __restrict__ y, const int* __restrict__ place, const float* __restrict__ weights, int top,
                   const TS* __restrict__ shared, int parts, size_t part_stride, const float* __restrict__ gate,
                   float* __restrict__ out, int H) {
    pdl_begin();
    const int t = blockIdx.x;
    for (int c = threadIdx.x; c < H; c += blockDim.x) {
        float v = 0.f;
        for (int k = 0; k < top; ++k) {
            const float term = weights[(size_t)t * top + k] * y[(size_t)place[(size_t)t * top + k] * H + c];
            v = k == 0 ? term : v + term;
        }
        if (shared != nullptr) {
            float s = 0.f;
            for (int p = 0; p < parts; ++p) {
                const float part = to_f32(shared[(size_t)p * part_stride + (size_t)t * H + c]);
                s = p == 0 ? part : s + part;
            }
            v = fmaf(gate[t], s, v);
        }
        out[(size_t)t * H + c] = v;
    }
}

WLLM_API int wllm_moe_route(const void* h, int dtype, const float* w_router, const float* w_gate, int* chosen, float* weights,
                            float* gate_out, int n, int H, int E, int top, int groups, int groups_kept, cudaStream_t stream) {
    if (n <= 0) return WLLM_OK;
    if (H <= 0 || E <= 0 || E > MOE_MAX_EXPERTS || top < 1 || groups < 1 || E % groups != 0 || groups_kept < 1 ||
        groups_kept > groups || top > groups_kept * (E / groups) || (w_gate != nullptr && gate_out == nullptr))
        return WLLM_BAD_SIZE;
    const size_t smem = (size_t)(H + E + groups) * sizeof(float);
    if (smem > 200 * 1024) return WLLM_BAD_SIZE;
#define GO(T) do { \
        if (smem > 48 * 1024) { \
            const cudaError_t er = cudaFuncSetAttribute(moe_route_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024); \
            if (er != cudaSuccess) return 1000 + (int)er; \
        } \
        return wllm_launch(moe_route_kernel<T>, n, 128, smem, stream, (const T*)h, w_router, w_gate, chosen, weights, gate_out, H, E, \
                           top, groups, groups_kept); \
    } while (0)
    if (dtype == WLLM_BF16) GO(bf16);
    if (dtype == WLLM_F32) GO(float);
#undef GO
    return WLLM_BAD_DTYPE;
}

// count [E], offset [E + 1], sorted [pairs], place [pairs]
WLLM_API int wllm_moe_plan(const int* chosen, int pairs, int E, int* count, int* offset, int* sorted, int* place, cudaStream_t stream) {
    if (pairs <= 0) return WLLM_OK;
    if (E <= 0 || E > MOE_MAX_EXPERTS) return WLLM_BAD_SIZE;
    const int st = wllm_launch(moe_count_kernel, (E + 3) / 4, 128, 0, stream, chosen, pairs, E, count);
    if (st != WLLM_OK) return st;
    return wllm_launch(moe_place_kernel, (E + 3) / 4, 128, 0, stream, chosen, pairs, E, (const int*)count, offset, sorted, place);
}

// gated = 1: a [n][K] rows of tokens (stride a_stride), w [E][2 N][K], out [pairs][N] of the operands' type;
// gated = 0: a [pairs][K] sorted rows, w [E][N][K], out [pairs][N] 32-bit.
WLLM_API int wllm_moe_grouped(const void* a, int a_stride, const void* w, void* out, int dtype, int gated, int pairs, int N, int K,
                              const int* offset, const int* sorted, int E, int top, float limit, float slope, cudaStream_t stream) {
    if (pairs <= 0) return WLLM_OK;
    if (N <= 0 || K <= 0 || E <= 0 || E > MOE_MAX_EXPERTS || top < 1) return WLLM_BAD_SIZE;
    const dim3 grid((N + GN - 1) / GN, (pairs + GM - 1) / GM + E);
    if (grid.y > 65535) return WLLM_BAD_SIZE;
#define GO(T, TO, G) wllm_launch(moe_grouped_kernel<T, TO, G>, grid, 256, 0, stream, (const T*)a, a_stride, (const T*)w, (TO*)out, N, K, \
                                 offset, sorted, E, top, limit, slope)
    if (dtype == WLLM_BF16) return gated ? GO(bf16, bf16, true) : GO(bf16, float, false);
    if (dtype == WLLM_F32) return gated ? GO(float, float, true) : GO(float, float, false);
#undef GO
    return WLLM_BAD_DTYPE;
}

WLLM_API int wllm_moe_combine(const float* y, const int* place, const float* weights, int top, const void* shared, int shared_dtype,
                              int parts, long long part_stride, const float* gate, float* out, int n, int H, cudaStream_t stream) {
    if (n <= 0) return WLLM_OK;
    if (H <= 0 || top < 1 || parts < 1 || (shared != nullptr && gate == nullptr)) return WLLM_BAD_SIZE;
    const int threads = H >= 1024 ? 256 : 128;
    if (shared == nullptr || shared_dtype == WLLM_F32)
        return wllm_launch(moe_combine_kernel<float>, n, threads, 0, stream, y, place, weights, top, (const float*)shared, parts,
                           (size_t)part_stride, gate, out, H);
    if (shared_dtype == WLLM_BF16 && parts == 1)
        return wllm_launch(moe_combine_kernel<bf16>, n, threads, 0, stream, y, place, weights, top, (const bf16*)shared, parts,
                           (size_t)part_stride, gate, out, H);
    return WLLM_BAD_DTYPE;
}
