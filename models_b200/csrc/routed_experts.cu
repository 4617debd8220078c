// A mixture of experts: every token uses the `top` experts with the largest router logits.
//
//   router:   z = R x (float sums), the `top` largest (ties to the lower index), weights = softmax over the chosen z
//   sort:     the (token, choice) entries grouped by expert, in token order, cut into tiles of 64 rows
//   expert e: g = min(Wg_e x, limit), u = clamp(Wu_e x, -limit, limit), y = Wd_e (g * sigmoid(slope * g) * (u + up_offset))
//             (limit +inf, slope 1, up_offset 0: the plain gated form silu(g) * u)
//   combine:  out[token] = sum_choice weight * y[token, choice] (+ sigmoid(score[token]) * shared[token])
//
// The two expert products are grouped products: a block owns one tile of one expert's rows and 64 output columns, reads
// that expert's weights, and gathers (first product) or scatters (second product) its rows by the sorted list, so a
// step of any size is three launches whose grids do not depend on how the router chose.  Every output is one chain of
// sums in ascending k: a row's result does not depend on what else is in the batch.  Storage float or bfloat16,
// arithmetic float; with bfloat16 storage and sizes that are multiples of 16 the products run on the tensor cores.
#include "common.cuh"

#include <math_constants.h>

MB_DEFINE_LAST_ERROR()

namespace mb {

constexpr int kTileRows = 64;
constexpr int kTileCols = 64;
constexpr int kMaxTop = 32;

__device__ __forceinline__ float sigmoid(float v) { return 1.0f / (1.0f + expf(-v)); }

__device__ __forceinline__ float clamped_swish(float g, float u, float limit, float slope, float up_offset) {
    g = fminf(g, limit);
    u = fminf(fmaxf(u, -limit), limit);
    return g * sigmoid(slope * g) * (u + up_offset);
}

// How a router turns logits into choices and weights.  scored == 0: the `top` largest logits, weights = softmax over the chosen
// logits.  scored != 0: scores s = softmax over ALL logits; the choice runs on s + correction (a float per expert, or null);
// the experts form `groups` equal groups of neighbours, a group counts by its largest choice score, and only experts of the
// `keep` best groups can be chosen (ties to the lower index everywhere); weights = weight_scale * s of the chosen, not
// renormalised.
struct RouterRule {
    int scored;
    const float* correction;
    int groups, keep;
    float weight_scale;
};

// grid (ceil(tokens / kTokens)); block 256.  shared per token of the block: width floats (its row), experts floats (its logits).
// kVector: width a multiple of 8 and rows on 16 (bfloat16) or 32 (float) bytes: a lane reads 8 elements of a router row with
// one or two wide loads, and a warp works on 4 experts at once so that as many loads are in flight.  kTokens > 1 (prompts):
// what a lane has loaded of the router serves so many tokens.  A token's sums are taken in the same order whatever kTokens is.
template <typename T, bool kVector, int kTokens>
__global__ void __launch_bounds__(256)
router_topk_kernel(const T* __restrict__ x, int x_stride, const T* __restrict__ router, int* __restrict__ chosen,
                   float* __restrict__ weights, int tokens, int width, int experts, int top, RouterRule rule) {
    grid_launch_dependents();
    grid_dependency_wait();
    extern __shared__ __align__(16) float router_shared[];
    float* rows = router_shared;                       // [kTokens][width]
    float* all_logits = router_shared + kTokens * width;  // [kTokens][experts]
    float* all_scores = all_logits + kTokens * experts;    // [kTokens][experts], a scored rule's softmax over all experts
    __shared__ float all_picked[kTokens][kMaxTop];
    const int token0 = blockIdx.x * kTokens, warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
    const int here = min(kTokens, tokens - token0);
    if (kVector) {
        for (int c = threadIdx.x; c < kTokens * (width / 8); c += blockDim.x) {
            const int t = c / (width / 8), piece = c % (width / 8);
            float v[8];
            load8(x + (size_t)min(token0 + t, tokens - 1) * x_stride + piece * 8, v);
#pragma unroll
            for (int i = 0; i < 8; ++i) rows[t * width + piece * 8 + i] = v[i];
        }
    } else {
        for (int c = threadIdx.x; c < width; c += blockDim.x) rows[c] = Num<T>::load(x + (size_t)token0 * x_stride + c);
    }
    __syncthreads();
    if (kVector) {
        constexpr int kAtOnce = 4;
        for (int e0 = warp * kAtOnce; e0 < experts; e0 += warps * kAtOnce) {
            float sum[kTokens][kAtOnce];
#pragma unroll
            for (int t = 0; t < kTokens; ++t)
#pragma unroll
                for (int j = 0; j < kAtOnce; ++j) sum[t][j] = 0.0f;
            for (int c = lane; c < width / 8; c += 32) {
                float w[kAtOnce][8];
#pragma unroll
                for (int j = 0; j < kAtOnce; ++j) load8(router + (size_t)min(e0 + j, experts - 1) * width + c * 8, w[j]);
#pragma unroll
                for (int t = 0; t < kTokens; ++t) {
                    const float4 x0 = *reinterpret_cast<const float4*>(rows + t * width + c * 8);
                    const float4 x1 = *reinterpret_cast<const float4*>(rows + t * width + c * 8 + 4);
                    const float xs[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
#pragma unroll
                    for (int j = 0; j < kAtOnce; ++j)
#pragma unroll
                        for (int i = 0; i < 8; ++i) sum[t][j] = fmaf(xs[i], w[j][i], sum[t][j]);
                }
            }
#pragma unroll
            for (int t = 0; t < kTokens; ++t)
#pragma unroll
                for (int j = 0; j < kAtOnce; ++j) {
                    const float total = warp_sum(sum[t][j]);
                    if (lane == 0 && e0 + j < experts) all_logits[t * experts + e0 + j] = total;
                }
        }
    } else {
        for (int e = warp; e < experts; e += warps) {
            const T* w = router + (size_t)e * width;
            float sum = 0.0f;
            for (int c = lane; c < width; c += 32) sum = fmaf(rows[c], Num<T>::load(w + c), sum);
            sum = warp_sum(sum);
            if (lane == 0) all_logits[e] = sum;
        }
    }
    __syncthreads();
    if (warp >= here) return;  // warp t picks for the block's token t
    const int token = token0 + warp;
    float* logits = all_logits + warp * experts;
    float* picked = all_picked[warp];
    if (rule.scored) {
        // scores over all experts, kept in `all_scores` for the weights; logits[e] becomes the choice score (-inf outside the
        // kept groups), on which the rounds of arg-max below run
        float top_logit = -CUDART_INF_F;
        for (int e = lane; e < experts; e += 32) top_logit = fmaxf(top_logit, logits[e]);
        top_logit = warp_max(top_logit);
        float sum = 0.0f;
        for (int e = lane; e < experts; e += 32) sum += expf(logits[e] - top_logit);
        sum = warp_sum(sum);
        float* scores = all_scores + warp * experts;
        for (int e = lane; e < experts; e += 32) {
            const float score = expf(logits[e] - top_logit) / sum;
            scores[e] = score;
            logits[e] = score + (rule.correction != nullptr ? rule.correction[e] : 0.0f);
        }
        __syncwarp();
        if (rule.groups > 1 && rule.keep < rule.groups) {
            // lane g finds group g's best choice score (groups <= 32); `keep` rounds pick the best groups; the others close
            const int per = experts / rule.groups;
            float group_best = -CUDART_INF_F;
            if (lane < rule.groups)
                for (int e = lane * per; e < (lane + 1) * per; ++e) group_best = fmaxf(group_best, logits[e]);
            bool kept = false;
            for (int round = 0; round < rule.keep; ++round) {
                float best = (lane < rule.groups && !kept) ? group_best : -CUDART_INF_F;
                int index = (lane < rule.groups && !kept) ? lane : 0x7fffffff;
#pragma unroll
                for (int offset = 16; offset > 0; offset >>= 1) {
                    const float other = __shfl_xor_sync(0xffffffffu, best, offset);
                    const int other_index = __shfl_xor_sync(0xffffffffu, index, offset);
                    if (other > best || (other == best && other_index < index)) best = other, index = other_index;
                }
                if (lane == index) kept = true;
            }
            const unsigned open = __ballot_sync(0xffffffffu, kept);
            for (int e = lane; e < experts; e += 32)
                if (!((open >> (e / per)) & 1u)) logits[e] = -CUDART_INF_F;
            __syncwarp();
        }
    }
    for (int s = 0; s < top; ++s) {
        // the largest logit that is not taken yet; ties go to the lower index (a taken expert's logit is -inf)
        float best = -CUDART_INF_F;
        int index = 0x7fffffff;
        for (int e = lane; e < experts; e += 32) {
            const float v = logits[e];
            if (v > best || (v == best && e < index)) best = v, index = e;
        }
#pragma unroll
        for (int offset = 16; offset > 0; offset >>= 1) {
            const float other = __shfl_xor_sync(0xffffffffu, best, offset);
            const int other_index = __shfl_xor_sync(0xffffffffu, index, offset);
            if (other > best || (other == best && other_index < index)) best = other, index = other_index;
        }
        if (index == 0x7fffffff) index = 0;  // (only if every logit is NaN)
        if (lane == 0) {
            chosen[(size_t)token * top + s] = index;
            picked[s] = best;
            logits[index] = -CUDART_INF_F;
        }
        __syncwarp();
    }
    __syncwarp();
    if (rule.scored) {
        const float* scores = all_scores + warp * experts;
        if (lane < top) weights[(size_t)token * top + lane] = rule.weight_scale * scores[chosen[(size_t)token * top + lane]];
        return;
    }
    if (lane == 0) {
        const float top_logit = picked[0];  // the largest: the first one picked
        float sum = 0.0f;
        for (int s = 0; s < top; ++s) sum += expf(picked[s] - top_logit);
        for (int s = 0; s < top; ++s) weights[(size_t)token * top + s] = expf(picked[s] - top_logit) / sum;
    }
}

// One block of 1024 threads.  entries = tokens * top.  offsets [experts + 1]; sorted [entries]: entry ids (token * top +
// choice) by expert, in ascending order within an expert; tile_expert / tile_row [max_tiles]: the expert (or -1) and the
// first row of the sorted list of every tile of kTileRows rows.
__global__ void __launch_bounds__(1024)
route_sort_kernel(const int* __restrict__ chosen, int entries, int experts, int* __restrict__ offsets, int* __restrict__ sorted,
                  int* __restrict__ tile_expert, int* __restrict__ tile_row, int max_tiles) {
    grid_launch_dependents();
    grid_dependency_wait();
    extern __shared__ int sort_shared[];  // counts [experts], starts [experts + 1]
    int* counts = sort_shared;
    int* starts = sort_shared + experts;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
    for (int e = warp; e < experts; e += warps) {
        int count = 0;
        for (int base = 0; base < entries; base += 32) {
            const int i = base + lane;
            count += __popc(__ballot_sync(0xffffffffu, i < entries && chosen[i] == e));
        }
        if (lane == 0) counts[e] = count;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int at = 0, tile = 0;
        for (int e = 0; e < experts; ++e) {
            starts[e] = at;
            offsets[e] = at;
            for (int r = 0; r < counts[e] && tile < max_tiles; r += kTileRows) {
                tile_expert[tile] = e;
                tile_row[tile] = at + r;
                ++tile;
            }
            at += counts[e];
        }
        starts[experts] = at;
        offsets[experts] = at;
        for (; tile < max_tiles; ++tile) tile_expert[tile] = -1, tile_row[tile] = 0;
    }
    __syncthreads();
    for (int e = warp; e < experts; e += warps) {
        int at = starts[e];
        for (int base = 0; base < entries; base += 32) {
            const int i = base + lane;
            const bool hit = i < entries && chosen[i] == e;
            const unsigned mask = __ballot_sync(0xffffffffu, hit);
            if (hit) sorted[at + __popc(mask & ((1u << lane) - 1u))] = i;
            at += __popc(mask);
        }
    }
}

// The same result for up to kFastExperts experts in three sweeps: every warp owns a stretch of the entries, counts its
// stretch per expert (lanes with the same expert find one another with a match), the counts become each warp's first place
// per expert, and the warp then puts its entries there in their order.  shared: counts [32][experts], totals [experts],
// starts [experts + 1].
constexpr int kFastExperts = 256;

__global__ void __launch_bounds__(1024)
route_sort_fast_kernel(const int* __restrict__ chosen, int entries, int experts, int* __restrict__ offsets, int* __restrict__ sorted,
                       int* __restrict__ tile_expert, int* __restrict__ tile_row, int max_tiles) {
    grid_launch_dependents();
    grid_dependency_wait();
    extern __shared__ int sort_shared[];
    int* counts = sort_shared;                 // [32][experts]
    int* totals = sort_shared + 32 * experts;  // [experts]
    int* starts = totals + experts;            // [experts + 1]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int i = threadIdx.x; i < 32 * experts; i += blockDim.x) counts[i] = 0;
    __syncthreads();
    const int stretch = ((entries + 32 * 32 - 1) / (32 * 32)) * 32;  // entries per warp, a multiple of 32
    const int first = warp * stretch, last = min(first + stretch, entries);
    int* mine = counts + warp * experts;
    for (int base = first; base < last; base += 32) {
        const int i = base + lane;
        int e = i < last ? chosen[i] : -1;
        if (e < 0 || e >= experts) e = -1;
        const unsigned same = __match_any_sync(0xffffffffu, e);
        if (e >= 0 && lane == __ffs(same) - 1) mine[e] += __popc(same);
        __syncwarp();
    }
    __syncthreads();
    for (int e = threadIdx.x; e < experts; e += blockDim.x) {
        int run = 0;
        for (int w = 0; w < 32; ++w) {
            const int count = counts[w * experts + e];
            counts[w * experts + e] = run;
            run += count;
        }
        totals[e] = run;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int at = 0, tile = 0;
        for (int e = 0; e < experts; ++e) {
            starts[e] = at;
            offsets[e] = at;
            for (int r = 0; r < totals[e] && tile < max_tiles; r += kTileRows) {
                tile_expert[tile] = e;
                tile_row[tile] = at + r;
                ++tile;
            }
            at += totals[e];
        }
        starts[experts] = at;
        offsets[experts] = at;
        for (; tile < max_tiles; ++tile) tile_expert[tile] = -1, tile_row[tile] = 0;
    }
    __syncthreads();
    for (int base = first; base < last; base += 32) {
        const int i = base + lane;
        int e = i < last ? chosen[i] : -1;
        if (e < 0 || e >= experts) e = -1;
        const unsigned same = __match_any_sync(0xffffffffu, e);
        if (e >= 0) sorted[starts[e] + mine[e] + __popc(same & ((1u << lane) - 1u))] = i;
        __syncwarp();
        if (e >= 0 && lane == __ffs(same) - 1) mine[e] += __popc(same);
        __syncwarp();
    }
}

// The entries by expert with every expert's rows starting on a multiple of kGroupTile rows, for products whose tiles of
// that many rows each belong to one expert.  One block of 1024 threads; up to kFastExperts experts (the sweeps of
// route_sort_fast_kernel).  sorted [max_tiles * kGroupTile]: the entry at every row, -1 at rows that only fill a tile up;
// position [entries]: the row of every entry; tile_group [max_tiles]: the expert of every tile, -1 past the last one.
constexpr int kGroupTile = 128;

__global__ void __launch_bounds__(1024)
route_pad_kernel(const int* __restrict__ chosen, int entries, int experts, int* __restrict__ sorted, int* __restrict__ position,
                 int* __restrict__ tile_group, int max_tiles, int staged) {
    grid_launch_dependents();
    grid_dependency_wait();
    extern __shared__ int sort_shared[];
    int* counts = sort_shared;                 // [32][experts]
    int* totals = sort_shared + 32 * experts;  // [experts]
    int* starts = totals + experts;            // [experts + 1]
    int* held = starts + experts + 1;          // [entries] if staged: every entry's expert (or -1), fetched once by all threads
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int i = threadIdx.x; i < 32 * experts; i += blockDim.x) counts[i] = 0;
    for (int i = threadIdx.x; i < max_tiles * kGroupTile; i += blockDim.x) sorted[i] = -1;
    if (staged) {
#pragma unroll 8
        for (int i = threadIdx.x; i < entries; i += blockDim.x) {  // (independent loads: many in flight per thread)
            const int e = chosen[i];
            held[i] = e < 0 || e >= experts ? -1 : e;
        }
    }
    __syncthreads();
    auto expert_of = [&](int i) {
        const int e = staged ? held[i] : chosen[i];
        return e < 0 || e >= experts ? -1 : e;
    };
    const int stretch = ((entries + 32 * 32 - 1) / (32 * 32)) * 32;
    const int first = warp * stretch, last = min(first + stretch, entries);
    int* mine = counts + warp * experts;
    for (int base = first; base < last; base += 32) {
        const int i = base + lane;
        const int e = i < last ? expert_of(i) : -1;
        const unsigned same = __match_any_sync(0xffffffffu, e);
        if (e >= 0 && lane == __ffs(same) - 1) mine[e] += __popc(same);
        __syncwarp();
    }
    __syncthreads();
    for (int e = threadIdx.x; e < experts; e += blockDim.x) {
        int run = 0;
        for (int w = 0; w < 32; ++w) {
            const int count = counts[w * experts + e];
            counts[w * experts + e] = run;
            run += count;
        }
        totals[e] = run;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int tile = 0;
        for (int e = 0; e < experts; ++e) {
            starts[e] = tile * kGroupTile;
            for (int r = 0; r < totals[e] && tile < max_tiles; r += kGroupTile) tile_group[tile++] = e;
        }
        for (; tile < max_tiles; ++tile) tile_group[tile] = -1;
    }
    __syncthreads();
    for (int base = first; base < last; base += 32) {
        const int i = base + lane;
        const int e = i < last ? expert_of(i) : -1;
        const unsigned same = __match_any_sync(0xffffffffu, e);
        if (e >= 0) {
            const int at = starts[e] + mine[e] + __popc(same & ((1u << lane) - 1u));
            sorted[at] = i;
            position[i] = at;
        }
        __syncwarp();
        if (e >= 0 && lane == __ffs(same) - 1) mine[e] += __popc(same);
        __syncwarp();
    }
    for (int i = first + lane; i < last; i += 32)  // (an entry whose expert does not exist reads row 0; its weight is what the router gave)
        if (expert_of(i) < 0) position[i] = 0;
}

// grid (max_tiles * kGroupTile); block 128.  out [row][K] = x [sorted[row] / top][K], zeros at rows that fill a tile up;
// rows of tiles past the last one are left as they are.  K a multiple of 8 bfloat16, rows on 16 bytes.
__global__ void __launch_bounds__(128)
gather_rows_kernel(const __nv_bfloat16* __restrict__ x, int x_stride, const int* __restrict__ sorted, const int* __restrict__ tile_group,
                   __nv_bfloat16* __restrict__ out, int top, int K) {
    grid_launch_dependents();
    grid_dependency_wait();
    const int row = blockIdx.x;
    if (tile_group[row / kGroupTile] < 0) return;
    const int entry = sorted[row];
    const uint4* src = entry >= 0 ? reinterpret_cast<const uint4*>(x + (size_t)(entry / top) * x_stride) : nullptr;
    uint4* dst = reinterpret_cast<uint4*>(out + (size_t)row * K);
    for (int c = threadIdx.x; c < K / 8; c += blockDim.x) dst[c] = src != nullptr ? src[c] : make_uint4(0u, 0u, 0u, 0u);
}

// The grouped product in plain float arithmetic.  grid (ceil(N / 64), max_tiles); block 256 (16 x 16; a thread 4 x 4).
// kFirst: a = x [tokens][K], rows gathered through the sorted list (token = entry / top); two weight sets [experts][N][K]
//         (gate, up); mid [entries][N] (sorted order) = clamped_swish(gate . x, up . x).
// else:   a = mid [entries][K] in sorted order; one weight set (down); slot_out [entry][N] (float), scattered by entry id.
template <typename T, bool kFirst>
__global__ void __launch_bounds__(256)
expert_product_kernel(const T* __restrict__ a, int a_stride, const T* __restrict__ w0, const T* __restrict__ w1,
                      T* __restrict__ mid, float* __restrict__ slot_out, int out_stride, const int* __restrict__ sorted,
                      const int* __restrict__ offsets, const int* __restrict__ tile_expert, const int* __restrict__ tile_row,
                      int top, int N, int K, float limit, float slope, float up_offset) {
    grid_launch_dependents();
    grid_dependency_wait();
    constexpr int kStep = 16;
    __shared__ float a_tile[kStep][kTileRows + 4];
    __shared__ float b_tile[kFirst ? 2 : 1][kStep][kTileCols + 4];
    __shared__ int source_row[kTileRows];
    const int expert = tile_expert[blockIdx.y];
    if (expert < 0) return;  // the whole block leaves
    const int row0 = tile_row[blockIdx.y];
    const int rows = min(kTileRows, offsets[expert + 1] - row0);
    const int n0 = blockIdx.x * kTileCols;
    if (threadIdx.x < kTileRows) {
        const int r = threadIdx.x;
        source_row[r] = r < rows ? (kFirst ? sorted[row0 + r] / top : row0 + r) : -1;
    }
    __syncthreads();
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    const int load_row = threadIdx.x >> 2, load_k = (threadIdx.x & 3) * 4;
    const T* w0_e = w0 + (size_t)expert * N * K;
    const T* w1_e = kFirst ? w1 + (size_t)expert * N * K : nullptr;
    float acc[kFirst ? 2 : 1][4][4];
#pragma unroll
    for (int s = 0; s < (kFirst ? 2 : 1); ++s)
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) acc[s][i][j] = 0.0f;
    for (int k0 = 0; k0 < K; k0 += kStep) {
        const int src = source_row[load_row];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int k = k0 + load_k + j;
            a_tile[load_k + j][load_row] = (src >= 0 && k < K) ? Num<T>::load(a + (size_t)src * a_stride + k) : 0.0f;
            const int n = n0 + load_row;
            b_tile[0][load_k + j][load_row] = (n < N && k < K) ? Num<T>::load(w0_e + (size_t)n * K + k) : 0.0f;
            if (kFirst) b_tile[kFirst ? 1 : 0][load_k + j][load_row] = (n < N && k < K) ? Num<T>::load(w1_e + (size_t)n * K + k) : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < kStep; ++kk) {
            const float4 av = *reinterpret_cast<const float4*>(&a_tile[kk][ty * 4]);
            const float ar[4] = {av.x, av.y, av.z, av.w};
#pragma unroll
            for (int s = 0; s < (kFirst ? 2 : 1); ++s) {
                const float4 bv = *reinterpret_cast<const float4*>(&b_tile[s][kk][tx * 4]);
                const float br[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
                for (int i = 0; i < 4; ++i)
#pragma unroll
                    for (int j = 0; j < 4; ++j) acc[s][i][j] = fmaf(ar[i], br[j], acc[s][i][j]);
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int r = ty * 4 + i;
        if (r >= rows) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n >= N) continue;
            if (kFirst)
                Num<T>::store(mid + (size_t)(row0 + r) * out_stride + n, clamped_swish(acc[0][i][j], acc[kFirst ? 1 : 0][i][j], limit, slope, up_offset));
            else
                slot_out[(size_t)sorted[row0 + r] * out_stride + n] = acc[0][i][j];
        }
    }
}

// Few entries (a decode step): no sorting and no tiles.  grid (ceil(N / 32), entries); block 256: the block's entry
// (token = entry / top, expert = chosen[entry]) is staged as floats in shared memory; a warp owns 4 of the block's 32
// columns, its lanes walk K in pieces of 8 elements (16-byte loads of the weights, 8 or 4 in flight per lane) and the sums
// meet in a shuffle.  Memory-bound: every matrix row is read once per entry that uses its expert.
// kFirst: a = x [tokens][K]; mid [entry][N] = clamped_swish(gate_e . x, up_e . x), rows in entry order.
// else:   a = mid [entries][K] in entry order; slot_out [entry][N] (float) = down_e . mid.
template <typename T, bool kFirst, bool kVector>
__global__ void __launch_bounds__(256)
expert_rows_kernel(const T* __restrict__ a, int a_stride, const T* __restrict__ w0, const T* __restrict__ w1, T* __restrict__ mid,
                   float* __restrict__ slot_out, int out_stride, const int* __restrict__ chosen, int top, int experts, int N, int K,
                   float limit, float slope, float up_offset) {
    grid_launch_dependents();
    grid_dependency_wait();
    constexpr int kCols = 4;
    constexpr int kSets = kFirst ? 2 : 1;
    extern __shared__ __align__(16) float rows_shared[];  // K floats
    const int entry = blockIdx.y;
    const int expert = chosen[entry];
    if (expert < 0 || expert >= experts) return;  // (a router that chose nothing real: nothing is written)
    const T* src = a + (size_t)(kFirst ? entry / top : entry) * a_stride;
    if (kVector) {
        for (int c = threadIdx.x; c < K / 8; c += blockDim.x) {
            float v[8];
            load8(src + c * 8, v);
#pragma unroll
            for (int i = 0; i < 8; ++i) rows_shared[c * 8 + i] = v[i];
        }
    } else {
        for (int c = threadIdx.x; c < K; c += blockDim.x) rows_shared[c] = Num<T>::load(src + c);
    }
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n0 = (blockIdx.x * 8 + warp) * kCols;
    if (n0 >= N) return;
    const T* w_e[kSets];
    w_e[0] = w0 + (size_t)expert * N * K;
    if (kFirst) w_e[kSets - 1] = w1 + (size_t)expert * N * K;
    float acc[kSets][kCols];
#pragma unroll
    for (int s = 0; s < kSets; ++s)
#pragma unroll
        for (int j = 0; j < kCols; ++j) acc[s][j] = 0.0f;
    if (kVector) {
        for (int c = lane; c < K / 8; c += 32) {
            float w[kSets][kCols][8];
#pragma unroll
            for (int s = 0; s < kSets; ++s)
#pragma unroll
                for (int j = 0; j < kCols; ++j) load8(w_e[s] + (size_t)min(n0 + j, N - 1) * K + c * 8, w[s][j]);
            const float4 x0 = *reinterpret_cast<const float4*>(rows_shared + c * 8);
            const float4 x1 = *reinterpret_cast<const float4*>(rows_shared + c * 8 + 4);
            const float x[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
#pragma unroll
            for (int s = 0; s < kSets; ++s)
#pragma unroll
                for (int j = 0; j < kCols; ++j)
#pragma unroll
                    for (int i = 0; i < 8; ++i) acc[s][j] = fmaf(x[i], w[s][j][i], acc[s][j]);
        }
    } else {
        for (int k = lane; k < K; k += 32) {
            const float x = rows_shared[k];
#pragma unroll
            for (int s = 0; s < kSets; ++s)
#pragma unroll
                for (int j = 0; j < kCols; ++j) acc[s][j] = fmaf(x, Num<T>::load(w_e[s] + (size_t)min(n0 + j, N - 1) * K + k), acc[s][j]);
        }
    }
#pragma unroll
    for (int s = 0; s < kSets; ++s)
#pragma unroll
        for (int j = 0; j < kCols; ++j) acc[s][j] = warp_sum(acc[s][j]);
    if (lane != 0) return;
#pragma unroll
    for (int j = 0; j < kCols; ++j) {
        const int n = n0 + j;
        if (n >= N) break;
        if (kFirst)
            Num<T>::store(mid + (size_t)entry * out_stride + n, clamped_swish(acc[0][j], acc[kSets - 1][j], limit, slope, up_offset));
        else
            slot_out[(size_t)entry * out_stride + n] = acc[0][j];
    }
}

// The same on the tensor cores: bfloat16, K a multiple of 16, rows of a and of the weights starting on 16 bytes.
// Block 128: warp w owns rows 16w .. 16w + 15 of the tile and all 64 columns; K in steps of 64 through two stages of
// cp.async copies (rows padded by 16 bytes so that ldmatrix reads without bank conflicts); m16n8k16 products, float sums.
namespace tc {

using bf16 = __nv_bfloat16;
constexpr int kStepK = 64;
constexpr int kRowBytes = kStepK * 2 + 16;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool valid) {
    const int bytes = valid ? 16 : 0;  // 0 source bytes: the 16 bytes are filled with zeros
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

template <bool kFirst>
__global__ void __launch_bounds__(128)
expert_product_tc_kernel(const bf16* __restrict__ a, int a_stride, const bf16* __restrict__ w0, const bf16* __restrict__ w1,
                         bf16* __restrict__ mid, float* __restrict__ slot_out, int out_stride, const int* __restrict__ sorted,
                         const int* __restrict__ offsets, const int* __restrict__ tile_expert, const int* __restrict__ tile_row,
                         int top, int N, int K, float limit, float slope, float up_offset) {
    grid_launch_dependents();
    grid_dependency_wait();
    constexpr int kSets = kFirst ? 2 : 1;
    constexpr int kTileBytes = kTileRows * kRowBytes;
    constexpr int kStageBytes = (1 + kSets) * kTileBytes;
    extern __shared__ __align__(16) unsigned char tc_smem[];
    __shared__ int source_row[kTileRows];
    const int expert = tile_expert[blockIdx.y];
    if (expert < 0) return;
    const int row0 = tile_row[blockIdx.y];
    const int rows = min(kTileRows, offsets[expert + 1] - row0);
    const int n0 = blockIdx.x * kTileCols;
    if (threadIdx.x < kTileRows) {
        const int r = threadIdx.x;
        source_row[r] = r < rows ? (kFirst ? sorted[row0 + r] / top : row0 + r) : -1;
    }
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, group_id = lane >> 2, tid4 = lane & 3;
    const bf16* w_e[kSets];
    w_e[0] = w0 + (size_t)expert * N * K;
    if (kFirst) w_e[kSets - 1] = w1 + (size_t)expert * N * K;
    const uint32_t base = smem_u32(tc_smem);
    const int steps = (K + kStepK - 1) / kStepK;
    auto load_stage = [&](int step, int stage) {
        const int k0 = step * kStepK;
        const uint32_t at = base + stage * kStageBytes;
        for (int i = threadIdx.x; i < kTileRows * 8; i += 128) {
            const int r = i >> 3, piece = i & 7;
            const int k = k0 + piece * 8;
            const int src = source_row[r];
            const bool a_ok = src >= 0 && k < K;
            cp_async16(at + r * kRowBytes + piece * 16, a_ok ? a + (size_t)src * a_stride + k : a, a_ok);
            const int n = n0 + r;
            const bool w_ok = n < N && k < K;
#pragma unroll
            for (int s = 0; s < kSets; ++s)
                cp_async16(at + (1 + s) * kTileBytes + r * kRowBytes + piece * 16, w_ok ? w_e[s] + (size_t)n * K + k : w_e[s], w_ok);
        }
    };
    float acc[kSets][8][4];
#pragma unroll
    for (int s = 0; s < kSets; ++s)
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) acc[s][nt][0] = acc[s][nt][1] = acc[s][nt][2] = acc[s][nt][3] = 0.0f;
    load_stage(0, 0);
    cp_async_commit();
    for (int step = 0; step < steps; ++step) {
        const int stage = step & 1;
        if (step + 1 < steps) {
            load_stage(step + 1, stage ^ 1);
            cp_async_commit();
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        const uint32_t a_at = base + stage * kStageBytes + (warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * kRowBytes + (lane >> 4) * 16;
#pragma unroll
        for (int ks = 0; ks < kStepK / 16; ++ks) {
            uint32_t af[4];
            ldmatrix_x4(af, a_at + ks * 32);
#pragma unroll
            for (int s = 0; s < kSets; ++s) {
                const uint32_t w_at = base + stage * kStageBytes + (1 + s) * kTileBytes;
#pragma unroll
                for (int part = 0; part < 4; ++part) {
                    uint32_t b[4];
                    const int w_row = part * 16 + (lane & 7) + ((lane >> 4) & 1) * 8;
                    ldmatrix_x4(b, w_at + w_row * kRowBytes + (ks * 2 + ((lane >> 3) & 1)) * 16);
                    mma_bf16(acc[s][2 * part], af, b[0], b[1]);
                    mma_bf16(acc[s][2 * part + 1], af, b[2], b[3]);
                }
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const int r = warp * 16 + group_id + 8 * half;
        if (r >= rows) continue;
        const size_t out_row = kFirst ? (size_t)(row0 + r) : (size_t)sorted[row0 + r];
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                const int n = n0 + nt * 8 + tid4 * 2 + c;
                if (n >= N) continue;
                const float v0 = acc[0][nt][2 * half + c];
                if (kFirst)
                    mid[out_row * out_stride + n] = __float2bfloat16_rn(clamped_swish(v0, acc[kSets - 1][nt][2 * half + c], limit, slope, up_offset));
                else
                    slot_out[out_row * out_stride + n] = v0;
            }
        }
    }
}

}  // namespace tc

// out[t][c] = clamped_swish(gate[t][c], up[t][c]); grid (ceil(rows * cols / 256)); block 256.
template <typename T>
__global__ void clamped_swish_kernel(const T* __restrict__ gate, const T* __restrict__ up, int in_stride, T* __restrict__ out,
                                     int out_stride, size_t total, int cols, float limit, float slope, float up_offset) {
    grid_launch_dependents();
    grid_dependency_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const size_t t = i / cols;
    const int c = (int)(i % cols);
    Num<T>::store(out + t * out_stride + c,
                  clamped_swish(Num<T>::load(gate + t * in_stride + c), Num<T>::load(up + t * in_stride + c), limit, slope, up_offset));
}

// out[t][c] = sum_s weights[t][s] * slot_out[t * top + s][c] (+ sigmoid(score[t]) * shared[t][c]); float out.
// `position` (or null): entry t * top + s has its row of slot_out at position[t * top + s] instead.
template <typename T>
__global__ void expert_combine_kernel(const float* __restrict__ slot_out, const float* __restrict__ weights,
                                      const float* __restrict__ shared, const T* __restrict__ score, int score_stride,
                                      float* __restrict__ out, size_t total, int width, int top, const int* __restrict__ position,
                                      const int* __restrict__ chosen, int experts, const T* __restrict__ rows, int rows_stride) {
    grid_launch_dependents();
    grid_dependency_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const size_t t = i / width;
    const int c = (int)(i % width);
    float sum = 0.0f;
    for (int s = 0; s < top; ++s) {
        if (chosen != nullptr && chosen[t * top + s] >= experts) {  // an identity expert: its result is the token's own row
            sum = fmaf(weights[t * top + s], Num<T>::load(rows + t * rows_stride + c), sum);
            continue;
        }
        const size_t row = position != nullptr ? (size_t)position[t * top + s] : t * top + s;  // where the entry's result lies
        sum = fmaf(weights[t * top + s], slot_out[row * width + c], sum);
    }
    if (shared != nullptr) sum = fmaf(score != nullptr ? sigmoid(Num<T>::load(score + t * score_stride)) : 1.0f, shared[i], sum);
    out[i] = sum;
}

// The same with four columns per thread (width a multiple of 4, rows on 16 bytes); every element's sum runs in the same order.
template <typename T>
__global__ void expert_combine_vec4_kernel(const float* __restrict__ slot_out, const float* __restrict__ weights,
                                           const float* __restrict__ shared, const T* __restrict__ score, int score_stride,
                                           float* __restrict__ out, size_t total4, int width, int top, const int* __restrict__ position,
                                           const int* __restrict__ chosen, int experts, const T* __restrict__ rows, int rows_stride) {
    grid_launch_dependents();
    grid_dependency_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total4) return;
    const int quads = width / 4;
    const size_t t = i / quads;
    const int c = (int)(i % quads) * 4;
    float4 sum = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    for (int s = 0; s < top; ++s) {
        const float w = weights[t * top + s];
        if (chosen != nullptr && chosen[t * top + s] >= experts) {  // an identity expert: its result is the token's own row
            const T* own = rows + t * rows_stride + c;
            sum.x = fmaf(w, Num<T>::load(own), sum.x); sum.y = fmaf(w, Num<T>::load(own + 1), sum.y);
            sum.z = fmaf(w, Num<T>::load(own + 2), sum.z); sum.w = fmaf(w, Num<T>::load(own + 3), sum.w);
            continue;
        }
        const size_t row = position != nullptr ? (size_t)position[t * top + s] : t * top + s;
        const float4 v = *reinterpret_cast<const float4*>(slot_out + row * width + c);
        sum.x = fmaf(w, v.x, sum.x); sum.y = fmaf(w, v.y, sum.y); sum.z = fmaf(w, v.z, sum.z); sum.w = fmaf(w, v.w, sum.w);
    }
    if (shared != nullptr) {
        const float g = score != nullptr ? sigmoid(Num<T>::load(score + t * score_stride)) : 1.0f;
        const float4 v = *reinterpret_cast<const float4*>(shared + t * width + c);
        sum.x = fmaf(g, v.x, sum.x); sum.y = fmaf(g, v.y, sum.y); sum.z = fmaf(g, v.z, sum.z); sum.w = fmaf(g, v.w, sum.w);
    }
    *reinterpret_cast<float4*>(out + t * width + c) = sum;
}

}  // namespace mb

using namespace mb;

MB_EXPORT int mb_route_tile_rows() { return kTileRows; }
MB_EXPORT int mb_route_max_top() { return kMaxTop; }

MB_EXPORT int mb_router_topk(const void* x, int x_stride, const void* router, int dtype, int* chosen, float* weights, int tokens,
                             int width, int experts, int top, int scored, const float* correction, int groups, int keep,
                             float weight_scale, cudaStream_t stream) {
    if (tokens <= 0) return 0;
    if (width <= 0 || experts <= 0 || top <= 0 || top > experts || top > kMaxTop)
        return fail("router_topk: width %d, %d experts, top %d (at most %d and the number of experts)", width, experts, top, kMaxTop);
    if (scored && (groups < 1 || groups > 32 || experts % groups || keep < 1 || keep > groups))
        return fail("router_topk: %d groups (at most 32, dividing the %d experts) of which %d are kept", groups, experts, keep);
    if (scored && top > (experts / groups) * keep) return fail("router_topk: top %d exceeds the %d experts of the kept groups", top, (experts / groups) * keep);
    const RouterRule rule{scored, correction, groups, keep, weight_scale};
    const size_t one = ((size_t)width + 2 * (size_t)experts) * sizeof(float);
    if (one > 200 * 1024) return fail("router_topk: a row of %d and %d logits exceed a block's shared memory", width, experts);
    const size_t unit = dtype == MB_F32 ? 32 : 16, element = dtype == MB_F32 ? 4 : 2;
    const bool vector = width % 8 == 0 && ((size_t)x_stride * element) % unit == 0 && !((uintptr_t)x % unit) && !((uintptr_t)router % unit);
    // tokens of a prompt that share what a block loads of the router: four, or eight where blocks of four would not all be
    // resident at once (the kernel is bound by a block's latency, so a second wave of blocks doubles its time)
    constexpr int kTogether = 4, kMany = 8;
    const bool together = vector && tokens >= 64 * kTogether && kTogether * one <= 200 * 1024;
    const bool many = together && (tokens + kTogether - 1) / kTogether > 2 * 148 && kMany * one <= 72 * 1024;
#define MB_ROUTER(T, VECTOR, TOKENS)                                                                                                  \
    do {                                                                                                                              \
        const size_t smem = TOKENS * one;                                                                                             \
        if (smem > 48 * 1024)                                                                                                         \
            cudaFuncSetAttribute(router_topk_kernel<T, VECTOR, TOKENS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);       \
        MB_LAUNCH("router_topk", (router_topk_kernel<T, VECTOR, TOKENS>), dim3((tokens + TOKENS - 1) / TOKENS), dim3(256), smem, stream, \
                  true, (const T*)x, x_stride, (const T*)router, chosen, weights, tokens, width, experts, top, rule);                       \
    } while (0)
    if (dtype == MB_F32) {
        if (many) MB_ROUTER(float, true, kMany); else if (together) MB_ROUTER(float, true, kTogether); else if (vector) MB_ROUTER(float, true, 1); else MB_ROUTER(float, false, 1);
    } else if (dtype == MB_BF16) {
        if (many) MB_ROUTER(__nv_bfloat16, true, kMany); else if (together) MB_ROUTER(__nv_bfloat16, true, kTogether); else if (vector) MB_ROUTER(__nv_bfloat16, true, 1); else MB_ROUTER(__nv_bfloat16, false, 1);
    } else {
        return fail("router_topk: unknown dtype code %d", dtype);
    }
#undef MB_ROUTER
    return 0;
}

MB_EXPORT int mb_route_max_tiles(int entries, int experts) { return (entries + kTileRows - 1) / kTileRows + experts; }

MB_EXPORT int mb_route_sort(const int* chosen, int entries, int experts, int* offsets, int* sorted, int* tile_expert, int* tile_row,
                            int max_tiles, cudaStream_t stream) {
    if (entries <= 0) return 0;
    if (experts <= 0 || experts > 4096) return fail("route_sort: %d experts (at most 4096)", experts);
    if (max_tiles < mb_route_max_tiles(entries, experts)) return fail("route_sort: room for %d tiles, %d may be needed", max_tiles, mb_route_max_tiles(entries, experts));
    if (experts <= kFastExperts) {
        MB_LAUNCH("route_sort", route_sort_fast_kernel, dim3(1), dim3(1024), (34 * (size_t)experts + 1) * sizeof(int), stream, true, chosen,
                  entries, experts, offsets, sorted, tile_expert, tile_row, max_tiles);
        return 0;
    }
    MB_LAUNCH("route_sort", route_sort_kernel, dim3(1), dim3(1024), (2 * (size_t)experts + 1) * sizeof(int), stream, true, chosen, entries,
              experts, offsets, sorted, tile_expert, tile_row, max_tiles);
    return 0;
}

MB_EXPORT int mb_route_group_tile() { return kGroupTile; }
MB_EXPORT int mb_route_pad_max_experts() { return kFastExperts; }
MB_EXPORT int mb_route_pad_max_tiles(int entries, int experts) { return (entries + kGroupTile - 1) / kGroupTile + experts; }

// sorted [max_tiles * 128], position [entries], tile_group [max_tiles]: see route_pad_kernel.
MB_EXPORT int mb_route_pad(const int* chosen, int entries, int experts, int* sorted, int* position, int* tile_group, int max_tiles,
                           cudaStream_t stream) {
    if (entries <= 0) return 0;
    if (experts <= 0 || experts > kFastExperts) return fail("route_pad: %d experts (at most %d)", experts, kFastExperts);
    if (max_tiles < mb_route_pad_max_tiles(entries, experts)) return fail("route_pad: room for %d tiles, %d may be needed", max_tiles, mb_route_pad_max_tiles(entries, experts));
    size_t smem = (34 * (size_t)experts + 1) * sizeof(int);
    const int staged = smem + (size_t)entries * sizeof(int) <= 160 * 1024 ? 1 : 0;  // the entries' experts in shared memory, if they fit
    if (staged) smem += (size_t)entries * sizeof(int);
    if (smem > 48 * 1024) {
        static size_t allowed = 0;  // (raised as needed; the attribute is per device context and function)
        if (smem > allowed) {
            if (cudaFuncSetAttribute(route_pad_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024 + 48 * 1024) != cudaSuccess)
                return fail("route_pad: cannot have %zu bytes of shared memory", smem);
            allowed = 208 * 1024;
        }
    }
    MB_LAUNCH("route_pad", route_pad_kernel, dim3(1), dim3(1024), smem, stream, true, chosen, entries, experts, sorted, position,
              tile_group, max_tiles, staged);
    return 0;
}

MB_EXPORT int mb_gather_rows(const void* x, int x_stride, const int* sorted, const int* tile_group, void* out, int rows, int top, int K,
                             cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (K <= 0 || K % 8 || x_stride % 8 || ((uintptr_t)x & 15) || ((uintptr_t)out & 15)) return fail("gather_rows: rows of %d elements (stride %d) must be multiples of 8 on 16-byte boundaries", K, x_stride);
    MB_LAUNCH("gather_rows", gather_rows_kernel, dim3(rows), dim3(128), 0, stream, true, (const __nv_bfloat16*)x, x_stride, sorted,
              tile_group, (__nv_bfloat16*)out, top, K);
    return 0;
}

// first != 0: a = x [tokens][K] gathered, w0 / w1 = gate / up [experts][N][K], mid [entries][N] written (storage type).
// first == 0: a = mid [entries][K], w0 = down [experts][N][K], slot_out [entries][N] (float) written by entry id.
MB_EXPORT int mb_expert_product(const void* a, int a_stride, const void* w0, const void* w1, void* mid, float* slot_out, int out_stride,
                                int dtype, const int* sorted, const int* offsets, const int* tile_expert, const int* tile_row,
                                int max_tiles, int top, int N, int K, float limit, float slope, float up_offset, int first, int tensor_cores,
                                cudaStream_t stream) {
    if (max_tiles <= 0) return 0;
    if (N <= 0 || K <= 0 || top <= 0) return fail("expert_product: N %d, K %d, top %d", N, K, top);
    if (max_tiles > 65535) return fail("expert_product: %d tiles exceed the grid limit 65535", max_tiles);
    const dim3 grid((N + kTileCols - 1) / kTileCols, max_tiles);
    if (tensor_cores && dtype == MB_BF16 && K % 8 == 0 && a_stride % 8 == 0 && !((uintptr_t)a & 15) && !((uintptr_t)w0 & 15) &&
        !((uintptr_t)w1 & 15)) {
        using namespace tc;
        if (first) {
            const size_t smem = 2 * 3 * (size_t)kTileRows * kRowBytes;
            static bool configured = false;
            if (!configured) {
                cudaError_t status = cudaFuncSetAttribute(expert_product_tc_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
                if (status != cudaSuccess) return fail("expert_product: cannot reserve %zu bytes of shared memory: %s", smem, cudaGetErrorString(status));
                configured = true;
            }
            MB_LAUNCH("expert_product_tc", expert_product_tc_kernel<true>, grid, dim3(128), smem, stream, true, (const bf16*)a, a_stride,
                      (const bf16*)w0, (const bf16*)w1, (bf16*)mid, slot_out, out_stride, sorted, offsets, tile_expert, tile_row, top, N, K, limit, slope, up_offset);
        } else {
            const size_t smem = 2 * 2 * (size_t)kTileRows * kRowBytes;
            static bool configured = false;
            if (!configured) {
                cudaError_t status = cudaFuncSetAttribute(expert_product_tc_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
                if (status != cudaSuccess) return fail("expert_product: cannot reserve %zu bytes of shared memory: %s", smem, cudaGetErrorString(status));
                configured = true;
            }
            MB_LAUNCH("expert_product_tc", expert_product_tc_kernel<false>, grid, dim3(128), smem, stream, true, (const bf16*)a, a_stride,
                      (const bf16*)w0, (const bf16*)w1, (bf16*)mid, slot_out, out_stride, sorted, offsets, tile_expert, tile_row, top, N, K, limit, slope, up_offset);
        }
        return 0;
    }
#define MB_PRODUCT(T, FIRST)                                                                                                        \
    MB_LAUNCH("expert_product", (expert_product_kernel<T, FIRST>), grid, dim3(256), 0, stream, true, (const T*)a, a_stride, (const T*)w0, \
              (const T*)w1, (T*)mid, slot_out, out_stride, sorted, offsets, tile_expert, tile_row, top, N, K, limit, slope, up_offset)
    if (dtype == MB_F32) {
        if (first) MB_PRODUCT(float, true); else MB_PRODUCT(float, false);
    } else if (dtype == MB_BF16) {
        if (first) MB_PRODUCT(__nv_bfloat16, true); else MB_PRODUCT(__nv_bfloat16, false);
    } else {
        return fail("expert_product: unknown dtype code %d", dtype);
    }
#undef MB_PRODUCT
    return 0;
}

// The products for few entries (see expert_rows_kernel); rows of mid and slot_out in entry order (token * top + choice).
MB_EXPORT int mb_expert_rows(const void* a, int a_stride, const void* w0, const void* w1, void* mid, float* slot_out, int out_stride,
                             int dtype, const int* chosen, int entries, int top, int experts, int N, int K, float limit, float slope, float up_offset,
                             int first, cudaStream_t stream) {
    if (entries <= 0) return 0;
    if (N <= 0 || K <= 0 || top <= 0 || experts <= 0) return fail("expert_rows: N %d, K %d, top %d, %d experts", N, K, top, experts);
    if (entries > 65535) return fail("expert_rows: %d entries exceed the grid limit 65535", entries);
    const size_t smem = (size_t)K * sizeof(float);
    if (smem > 200 * 1024) return fail("expert_rows: a row of %d elements exceeds a block's shared memory", K);
    const dim3 grid((N + 31) / 32, entries);
    const size_t unit = dtype == MB_F32 ? 32 : 16;
    const size_t element = dtype == MB_F32 ? 4 : 2;
    const bool vector = K % 8 == 0 && ((size_t)a_stride * element) % unit == 0 && !((uintptr_t)a % unit) && !((uintptr_t)w0 % unit) &&
                        !((uintptr_t)w1 % unit);
#define MB_ROWS(T, FIRST, VECTOR)                                                                                                    \
    do {                                                                                                                             \
        if (smem > 48 * 1024) cudaFuncSetAttribute(expert_rows_kernel<T, FIRST, VECTOR>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        MB_LAUNCH("expert_rows", (expert_rows_kernel<T, FIRST, VECTOR>), grid, dim3(256), smem, stream, true, (const T*)a, a_stride,  \
                  (const T*)w0, (const T*)w1, (T*)mid, slot_out, out_stride, chosen, top, experts, N, K, limit, slope, up_offset);               \
    } while (0)
#define MB_ROWS_OF(T)                                                              \
    do {                                                                           \
        if (first && vector) MB_ROWS(T, true, true);                               \
        else if (first) MB_ROWS(T, true, false);                                   \
        else if (vector) MB_ROWS(T, false, true);                                  \
        else MB_ROWS(T, false, false);                                             \
    } while (0)
    if (dtype == MB_F32) MB_ROWS_OF(float);
    else if (dtype == MB_BF16) MB_ROWS_OF(__nv_bfloat16);
    else return fail("expert_rows: unknown dtype code %d", dtype);
#undef MB_ROWS_OF
#undef MB_ROWS
    return 0;
}

MB_EXPORT int mb_clamped_swish(const void* gate, const void* up, int in_stride, void* out, int out_stride, int dtype, int rows, int cols,
                               float limit, float slope, float up_offset, cudaStream_t stream) {
    if (rows <= 0 || cols <= 0) return 0;
    const size_t total = (size_t)rows * cols;
    const dim3 grid((unsigned)((total + 255) / 256));
    if (dtype == MB_F32)
        MB_LAUNCH("clamped_swish", clamped_swish_kernel<float>, grid, dim3(256), 0, stream, true, (const float*)gate, (const float*)up, in_stride,
                  (float*)out, out_stride, total, cols, limit, slope, up_offset);
    else if (dtype == MB_BF16)
        MB_LAUNCH("clamped_swish", clamped_swish_kernel<__nv_bfloat16>, grid, dim3(256), 0, stream, true, (const __nv_bfloat16*)gate,
                  (const __nv_bfloat16*)up, in_stride, (__nv_bfloat16*)out, out_stride, total, cols, limit, slope, up_offset);
    else
        return fail("clamped_swish: unknown dtype code %d", dtype);
    return 0;
}

// shared may be null (no shared expert); score (or null: the shared expert is added as it is) is one number per token of the
// storage type `dtype` (stride in elements).  With `chosen` [tokens * top], an entry whose expert is >= `experts` is an identity
// expert: its result is the token's own row of `rows` (storage type, stride in elements).
MB_EXPORT int mb_expert_combine(const float* slot_out, const float* weights, const float* shared, const void* score, int score_stride,
                                int dtype, float* out, int tokens, int width, int top, const int* position, const int* chosen,
                                int experts, const void* rows, int rows_stride, cudaStream_t stream) {
    if (tokens <= 0 || width <= 0) return 0;
    if (chosen != nullptr && rows == nullptr) return fail("expert_combine: identity experts need the tokens' rows");
    const size_t total = (size_t)tokens * width;
    if (dtype != MB_F32 && dtype != MB_BF16) return fail("expert_combine: unknown dtype code %d", dtype);
    if (width % 4 == 0 && !((uintptr_t)slot_out & 15) && !((uintptr_t)out & 15) && !((uintptr_t)shared & 15)) {
        const size_t total4 = total / 4;
        const dim3 grid4((unsigned)((total4 + 255) / 256));
        if (dtype == MB_F32)
            MB_LAUNCH("expert_combine", expert_combine_vec4_kernel<float>, grid4, dim3(256), 0, stream, true, slot_out, weights, shared,
                      (const float*)score, score_stride, out, total4, width, top, position, chosen, experts, (const float*)rows, rows_stride);
        else
            MB_LAUNCH("expert_combine", expert_combine_vec4_kernel<__nv_bfloat16>, grid4, dim3(256), 0, stream, true, slot_out, weights, shared,
                      (const __nv_bfloat16*)score, score_stride, out, total4, width, top, position, chosen, experts, (const __nv_bfloat16*)rows, rows_stride);
        return 0;
    }
    const dim3 grid((unsigned)((total + 255) / 256));
    if (dtype == MB_F32)
        MB_LAUNCH("expert_combine", expert_combine_kernel<float>, grid, dim3(256), 0, stream, true, slot_out, weights, shared, (const float*)score,
                  score_stride, out, total, width, top, position, chosen, experts, (const float*)rows, rows_stride);
    else if (dtype == MB_BF16)
        MB_LAUNCH("expert_combine", expert_combine_kernel<__nv_bfloat16>, grid, dim3(256), 0, stream, true, slot_out, weights, shared,
                  (const __nv_bfloat16*)score, score_stride, out, total, width, top, position, chosen, experts, (const __nv_bfloat16*)rows, rows_stride);
    else
        return fail("expert_combine: unknown dtype code %d", dtype);
    return 0;
}
