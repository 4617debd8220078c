// The tensor-core form of csrc/gated_attention.cu for steps of many tokens: bfloat16 storage, cache pages of 64
// positions, key and value sizes fixed at compile time (-DMB_KEY_DIM, -DMB_VALUE_DIM: multiples of 16 up to 256;
// -DMB_SHARED_ROWS=1: the values are the key rows themselves, so a page is copied once and read as both).
//
//   score(i, j) = scale * q_h(i) . k_c(j) - slope_h * (i - j) + bias_h,   weight: softmax over j <= i, or sigmoid
//   out_h(i) = gate * sum_j weight(i, j) v_c(j)
//
// and the same variations of the score as there (ScoreExtras: a factor per head, a bound cap * tanh(. / cap), a sink in
// the softmax's denominator, a result whose pairs (2m, 2m + 1) are turned back by the query's position).
//
// A block owns 64 query tokens of one head (a warp 16 of them) and walks the pages of keys up to its last token
// through two stages of cp.async copies.  Scores are m16n8k16 products with float accumulators; slope, bias, mask,
// sigmoid or running softmax are float arithmetic on them.  The weights stay float: a tensor-core operand is bfloat16,
// so every weight goes into the product with the values as two numbers, its bfloat16 rounding and the bfloat16
// rounding of what that left over (together about 16 bits of the float weight, accumulated in float).
#include "common.cuh"

#include <math_constants.h>

#if !defined(MB_KEY_DIM) || !defined(MB_VALUE_DIM)
#error "compile with -DMB_KEY_DIM=<key size> -DMB_VALUE_DIM=<value size>"
#endif
#ifndef MB_SHARED_ROWS
#define MB_SHARED_ROWS 0
#endif

MB_DEFINE_LAST_ERROR()

namespace mb {

constexpr int KD = MB_KEY_DIM, VD = MB_VALUE_DIM;
constexpr bool kSharedRows = MB_SHARED_ROWS != 0;
static_assert(KD % 16 == 0 && KD >= 16 && KD <= 256, "key size must be a multiple of 16 in 16..256");
static_assert(VD % 16 == 0 && VD >= 16 && VD <= 256, "value size must be a multiple of 16 in 16..256");
static_assert(!kSharedRows || VD <= KD, "values read from key rows cannot be wider than the rows");
constexpr int kTile = 64;  // keys per tile, one cache page
constexpr int kQRows = 64;
constexpr int kThreads = 128;
constexpr int kKeyRow = KD * 2 + 16;  // padded shared-memory rows: ldmatrix reads without bank conflicts
constexpr int kValueRow = kSharedRows ? kKeyRow : VD * 2 + 16;
constexpr int kKeyTile = kTile * kKeyRow;
constexpr int kStageBytes = kKeyTile + (kSharedRows ? 0 : kTile * kValueRow);
constexpr int kKSteps = KD / 16;
constexpr bool kKeepQueries = KD <= 128;  // query fragments in registers; beyond that they are read from shared memory per step
constexpr int kGateHead = 1, kGateElement = 2;

using bf16 = __nv_bfloat16;

struct ScoreExtras {
    const float* head_scale;  // [heads] factors on the scaled product, or null
    float softcap;            // 0: scores are not bounded
    int sink;                 // != 0: the softmax's denominator has one more term of score 0
    const float* turn_cos;    // [positions][VD / 2] with turn_sin: the result's pairs are turned by minus the query's position
    const float* turn_sin;
    int block;                // n > 0: a query sees only the keys of its own block of n positions (counted from 0); 0: every earlier key
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(dst), "l"(src));
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
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float quad_max(float v) {
    v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 1));
    return fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 2));
}
__device__ __forceinline__ float quad_sum(float v) {
    v += __shfl_xor_sync(0xffffffffu, v, 1);
    return v + __shfl_xor_sync(0xffffffffu, v, 2);
}

// Two float weights as a pair of bfloat16 roundings and the pair of what the roundings left over.
__device__ __forceinline__ void split_pair(float a, float b, uint32_t& hi, uint32_t& lo) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    const float2 back = __bfloat1622float2(h);
    const __nv_bfloat162 l = __floats2bfloat162_rn(a - back.x, b - back.y);
    hi = *reinterpret_cast<const uint32_t*>(&h);
    lo = *reinterpret_cast<const uint32_t*>(&l);
}

// One page of one kv head ([64][kDim] contiguous in the pool) -> a padded tile in shared memory (all threads).
template <int kDim, int kRow>
__device__ __forceinline__ void load_tile(uint32_t dst, const bf16* __restrict__ pool, size_t page, int kv_head, int kv_heads) {
    constexpr int kPieces = kDim / 8;
    const bf16* src = pool + (page * kv_heads + kv_head) * (size_t)(kTile * kDim);
#pragma unroll
    for (int j = 0; j < kTile * kPieces / kThreads; ++j) {
        const int i = threadIdx.x + j * kThreads;
        const int row = i / kPieces, piece = i % kPieces;
        cp_async16(dst + row * kRow + piece * 16, src + row * kDim + piece * 8);
    }
}

__device__ __forceinline__ void load_stage(uint32_t dst, const bf16* __restrict__ k_pool, const bf16* __restrict__ v_pool,
                                           size_t page, int kv_head, int kv_heads) {
    load_tile<KD, kKeyRow>(dst, k_pool, page, kv_head, kv_heads);
    if (!kSharedRows) load_tile<VD, kValueRow>(dst + kKeyTile, v_pool, page, kv_head, kv_heads);
}

// grid (query tiles of 64 tokens, heads, sequences); warp w owns tokens 16w..16w+15 of the tile.
template <bool kSoftmax>
__global__ void __launch_bounds__(kThreads)
gated_attention_tc_kernel(const bf16* __restrict__ q, int q_stride, bf16* __restrict__ out, int out_stride,
                          const bf16* __restrict__ k_pool, const bf16* __restrict__ v_pool, const int* __restrict__ block_table,
                          int max_blocks, const int* __restrict__ cu_q, const int* __restrict__ kv_lens,
                          const float* __restrict__ head_bias, const bf16* __restrict__ gate, int gate_stride, int gate_kind,
                          int heads, int kv_heads, float scale, float slope_exponent, ScoreExtras extras) {
    grid_launch_dependents();
    grid_dependency_wait();
    extern __shared__ __align__(16) unsigned char smem[];
    unsigned char* q_smem = smem;                      // 64 rows of queries
    unsigned char* stage_smem = smem + kQRows * kKeyRow;  // 2 stages x (key tile, value tile)
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, group_id = lane >> 2, tid4 = lane & 3;
    const int seq = blockIdx.z, head = blockIdx.y;
    const int kv_head = head / (heads / kv_heads);
    const int q_begin = cu_q[seq];
    const int q_len = cu_q[seq + 1] - q_begin;
    const int q_tile = gridDim.x - 1 - blockIdx.x;  // the tiles with the most keys start first
    const int t0 = q_tile * kQRows;
    if (t0 >= q_len) return;
    const int valid = min(kQRows, q_len - t0);
    const int kv_len = kv_lens[seq];
    const int pos0 = kv_len - q_len + t0;  // position of the tile's first token
    const int last_pos = pos0 + valid - 1;
    const int t_end = last_pos / kTile + 1;
    // with blocks of visibility the first position any row of the tile sees is the lowest row's (the bound grows with the position)
    const int t_begin = extras.block > 0 ? ((pos0 / extras.block) * extras.block) / kTile : 0;
    const float slope = slope_exponent != 0.0f ? exp2f(-slope_exponent * (float)(head + 1) / (float)heads) : 0.0f;
    const float bias = head_bias != nullptr ? head_bias[head] : 0.0f;
    constexpr float kLog2e = 1.4426950408889634f;
    if (extras.head_scale != nullptr) scale *= extras.head_scale[head];
    const float cap = extras.softcap;
    const float cap_exponent = cap > 0.0f ? 2.0f * kLog2e / cap : 0.0f;

    const int* table = block_table + (size_t)seq * max_blocks;
    const uint32_t stage_base = smem_u32(stage_smem);
    load_stage(stage_base + (t_begin & 1) * kStageBytes, k_pool, v_pool, table[t_begin], kv_head, kv_heads);
    cp_async_commit();
    {
        constexpr int kPieces = KD / 8;
        const bf16* first = q + (size_t)(q_begin + t0) * q_stride + (size_t)head * KD;
        for (int i = threadIdx.x; i < kQRows * kPieces; i += kThreads) {
            const int row = i / kPieces, piece = i % kPieces;
            uint4 v = make_uint4(0u, 0u, 0u, 0u);
            if (row < valid) v = *reinterpret_cast<const uint4*>(first + (size_t)row * q_stride + piece * 8);
            *reinterpret_cast<uint4*>(q_smem + row * kKeyRow + piece * 16) = v;
        }
    }
    __syncthreads();
    const uint32_t q_rows = smem_u32(q_smem) + warp * 16 * kKeyRow + ((lane & 7) + ((lane >> 3) & 1) * 8) * kKeyRow + (lane >> 4) * 16;
    uint32_t a_kept[kKeepQueries ? kKSteps : 1][4];
    if (kKeepQueries) {
#pragma unroll
        for (int ks = 0; ks < kKSteps; ++ks) ldmatrix_x4(a_kept[kKeepQueries ? ks : 0], q_rows + ks * 32);
    }

    float o[VD / 8][4];
#pragma unroll
    for (int i = 0; i < VD / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f;
    float run_max[2] = {-CUDART_INF_F, -CUDART_INF_F}, run_sum[2] = {0.0f, 0.0f};
    if (kSoftmax && extras.sink) {  // a key of score 0 whose value is zero, there before the first tile; one lane of four counts it
        run_max[0] = run_max[1] = 0.0f;
        run_sum[0] = run_sum[1] = tid4 == 0 ? 1.0f : 0.0f;
    }
    int row_pos[2], row_low[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int row = warp * 16 + group_id + 8 * r;
        row_pos[r] = row < valid ? pos0 + row : -1;  // a row beyond the sequence sees nothing
        row_low[r] = extras.block > 0 && row < valid ? (row_pos[r] / extras.block) * extras.block : 0;
    }
    const int warp_last = min(pos0 + warp * 16 + 15, last_pos);  // highest position among the warp's rows
    const int warp_first_pos = pos0 + warp * 16;                  // lowest
    const bool warp_has_rows = warp * 16 < valid;
    const int warp_first_low = extras.block > 0 ? (warp_first_pos / extras.block) * extras.block : 0;  // lowest first-visible position
    const int warp_low = extras.block > 0 ? (warp_last / extras.block) * extras.block : 0;  // highest first-visible position among the warp's rows

    for (int t = t_begin; t < t_end; ++t) {
        const int stage = t & 1;
        if (t + 1 < t_end) {
            load_stage(stage_base + (stage ^ 1) * kStageBytes, k_pool, v_pool, table[t + 1], kv_head, kv_heads);
            cp_async_commit();
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        const uint32_t k_tile = stage_base + stage * kStageBytes;
        const uint32_t v_tile = kSharedRows ? k_tile : k_tile + kKeyTile;
        const int key_base = t * kTile;
        if (key_base + kTile > kv_len) {
            // The sequence ends inside this page: the rows beyond its end hold whatever the page's last owner left.
            // Their weights are 0, but 0 times a stray infinity or NaN is NaN, so the value rows are cleared.
            unsigned char* rows = stage_smem + stage * kStageBytes + (kSharedRows ? 0 : kKeyTile);
            constexpr int kPieces = kValueRow / 16;
            const int first_stale = kv_len - key_base;
            for (int i = threadIdx.x; i < (kTile - first_stale) * kPieces; i += kThreads)
                *reinterpret_cast<uint4*>(rows + (first_stale + i / kPieces) * kValueRow + (i % kPieces) * 16) = make_uint4(0u, 0u, 0u, 0u);
            __syncthreads();
        }
        if (t == t_begin && extras.block > 0) {
            // The first tile may begin before the first key that any row of this block sees.  Those rows have weight 0 for
            // every query, but 0 times a stray infinity or NaN is NaN, so their value rows are cleared too.
            const int unseen = (pos0 / extras.block) * extras.block - key_base;
            if (unseen > 0) {
                unsigned char* rows = stage_smem + stage * kStageBytes + (kSharedRows ? 0 : kKeyTile);
                constexpr int kPieces = kValueRow / 16;
                if (!kSharedRows) {
                    for (int i = threadIdx.x; i < unseen * kPieces; i += kThreads)
                        *reinterpret_cast<uint4*>(rows + (i / kPieces) * kValueRow + (i % kPieces) * 16) = make_uint4(0u, 0u, 0u, 0u);
                    __syncthreads();
                }
            }
        }
        if (warp_has_rows && key_base <= warp_last && key_base + kTile > warp_first_low) {
            const bool full = key_base + kTile - 1 <= warp_first_pos && warp * 16 + 15 < valid && key_base >= warp_low;  // no mask needed
            float s[kTile / 8][4];
#pragma unroll
            for (int part = 0; part < kTile / 16; ++part) {
#pragma unroll
                for (int i = 0; i < 4; ++i) s[2 * part][i] = s[2 * part + 1][i] = 0.0f;
                const int key = part * 16 + (lane & 7) + ((lane >> 4) & 1) * 8;
#pragma unroll
                for (int ks = 0; ks < kKSteps; ++ks) {
                    uint32_t a_now[4], b[4];
                    if (!kKeepQueries) ldmatrix_x4(a_now, q_rows + ks * 32);
                    ldmatrix_x4(b, k_tile + key * kKeyRow + (ks * 2 + ((lane >> 3) & 1)) * 16);
                    mma_bf16(s[2 * part], kKeepQueries ? a_kept[kKeepQueries ? ks : 0] : a_now, b[0], b[1]);
                    mma_bf16(s[2 * part + 1], kKeepQueries ? a_kept[kKeepQueries ? ks : 0] : a_now, b[2], b[3]);
                }
            }
            // score = scale * q.k - slope * (i - j) + bias, all float; an invisible key gets weight 0
            float part_max[2] = {-CUDART_INF_F, -CUDART_INF_F};
#pragma unroll
            for (int nt = 0; nt < kTile / 8; ++nt)
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int key = key_base + nt * 8 + tid4 * 2 + (i & 1);
                    const int r = i >> 1;
                    float z = fmaf(s[nt][i], scale, bias) - slope * (float)(row_pos[r] - key);
                    // cap * tanh(z / cap) with tanh(x) = 1 - 2 / (1 + e^(2x))
                    if (cap > 0.0f) z = cap - __fdividef(2.0f * cap, 1.0f + fast_exp2(z * cap_exponent));
                    if (!full && (key > row_pos[r] || key < row_low[r])) z = -CUDART_INF_F;
                    if (kSoftmax) {
                        part_max[r] = fmaxf(part_max[r], z);
                        s[nt][i] = z;
                    } else {
                        s[nt][i] = __fdividef(1.0f, 1.0f + fast_exp2(-z * kLog2e));  // sigmoid; 1 / (1 + 2^inf) = 0
                    }
                }
            if (kSoftmax) {
#pragma unroll
                for (int r = 0; r < 2; ++r) {
                    const float new_max = fmaxf(run_max[r], quad_max(part_max[r]));
                    const float safe_max = new_max == -CUDART_INF_F ? 0.0f : new_max;  // a row that has seen nothing yet
                    const float correction = fast_exp2((run_max[r] - safe_max) * kLog2e);
                    run_max[r] = new_max;
                    float local = 0.0f;
#pragma unroll
                    for (int nt = 0; nt < kTile / 8; ++nt)
#pragma unroll
                        for (int c = 0; c < 2; ++c) {
                            const float e = fast_exp2((s[nt][2 * r + c] - safe_max) * kLog2e);
                            s[nt][2 * r + c] = e;
                            local += e;
                        }
                    run_sum[r] = run_sum[r] * correction + local;
#pragma unroll
                    for (int i = 0; i < VD / 8; ++i) {
                        o[i][2 * r] *= correction;
                        o[i][2 * r + 1] *= correction;
                    }
                }
            }
#pragma unroll
            for (int part = 0; part < kTile / 16; ++part) {
                uint32_t hi[4], lo[4];
                split_pair(s[2 * part][0], s[2 * part][1], hi[0], lo[0]);
                split_pair(s[2 * part][2], s[2 * part][3], hi[1], lo[1]);
                split_pair(s[2 * part + 1][0], s[2 * part + 1][1], hi[2], lo[2]);
                split_pair(s[2 * part + 1][2], s[2 * part + 1][3], hi[3], lo[3]);
                const int key = part * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
#pragma unroll
                for (int dp = 0; dp < VD / 16; ++dp) {
                    uint32_t b[4];
                    ldmatrix_x4_trans(b, v_tile + key * kValueRow + (dp * 2 + (lane >> 4)) * 16);
                    mma_bf16(o[2 * dp], hi, b[0], b[1]);
                    mma_bf16(o[2 * dp + 1], hi, b[2], b[3]);
                    mma_bf16(o[2 * dp], lo, b[0], b[1]);
                    mma_bf16(o[2 * dp + 1], lo, b[2], b[3]);
                }
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int row = warp * 16 + group_id + 8 * r;
        const float total = kSoftmax ? quad_sum(run_sum[r]) : 1.0f;
        if (row >= valid) continue;
        const size_t token = (size_t)(q_begin + t0 + row);
        float factor = kSoftmax ? 1.0f / total : 1.0f;
        if (gate_kind == kGateHead) factor *= 1.0f / (1.0f + expf(-__bfloat162float(gate[token * gate_stride + head])));
        bf16* out_row = out + token * out_stride + (size_t)head * VD;
        const size_t turn_at = extras.turn_cos != nullptr ? (size_t)row_pos[r] * (VD / 2) : 0;
#pragma unroll
        for (int i = 0; i < VD / 8; ++i) {
            const int d = i * 8 + tid4 * 2;
            float x = o[i][2 * r] * factor, y = o[i][2 * r + 1] * factor;
            if (extras.turn_cos != nullptr) {
                const float c = extras.turn_cos[turn_at + d / 2], sn = extras.turn_sin[turn_at + d / 2];
                const float x0 = x;
                x = x0 * c + y * sn;
                y = y * c - x0 * sn;
            }
            if (gate_kind == kGateElement) {
                const float2 g = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(gate + token * gate_stride + (size_t)head * VD + d));
                x *= 1.0f / (1.0f + expf(-g.x));
                y *= 1.0f / (1.0f + expf(-g.y));
            }
            *reinterpret_cast<__nv_bfloat162*>(out_row + d) = __floats2bfloat162_rn(x, y);
        }
    }
}

constexpr size_t kSmemBytes = (size_t)kQRows * kKeyRow + 2 * (size_t)kStageBytes;

}  // namespace mb

using namespace mb;

MB_EXPORT int mb_gated_attention_tc_key_dim() { return KD; }
MB_EXPORT int mb_gated_attention_tc_value_dim() { return VD; }

// q rows of `heads` heads of KD (stride in elements, a multiple of 8, 16-byte aligned); out rows of `heads` heads of VD
// (stride and start even); gate (if any) with even stride and start.  softmax != 0: softmax weights, else sigmoids.
MB_EXPORT int mb_gated_attention_tc(const void* q, int q_stride, void* out, int out_stride, const void* k_pool, const void* v_pool,
                                    const int* block_table, int max_blocks, const int* cu_q, const int* kv_lens,
                                    const float* head_bias, const void* gate, int gate_stride, int gate_kind, int sequences,
                                    int max_q_len, int heads, int kv_heads, int page_size, int softmax, float scale,
                                    float slope_exponent, const float* head_scale, float softcap, int sink, const float* turn_cos,
                                    const float* turn_sin, int block, cudaStream_t stream) {
    if (sequences <= 0 || max_q_len <= 0) return 0;
    if ((turn_cos == nullptr) != (turn_sin == nullptr)) return fail("gated_attention_tc: turning the result back needs both tables");
    if (softcap < 0.0f || (sink && !softmax)) return fail("gated_attention_tc: softcap %g, a sink without a softmax", softcap);
    const ScoreExtras extras{head_scale, softcap, sink, turn_cos, turn_sin, block};
    if (page_size != kTile) return fail("gated_attention_tc: cache pages must hold %d positions, got %d", kTile, page_size);
    if (kv_heads <= 0 || heads % kv_heads) return fail("gated_attention_tc: %d heads are no multiple of %d kv heads", heads, kv_heads);
    if (sequences > 65535 || heads > 65535) return fail("gated_attention_tc: %d sequences or %d heads exceed the grid limit 65535", sequences, heads);
    if (q_stride % 8 || ((uintptr_t)q & 15) || out_stride % 2 || ((uintptr_t)out & 3) || ((uintptr_t)k_pool & 15) || ((uintptr_t)v_pool & 15))
        return fail("gated_attention_tc: query rows must start on 16 bytes and result rows on 4");
    if (gate_kind < 0 || gate_kind > 2 || (gate_kind != 0 && gate == nullptr)) return fail("gated_attention_tc: gate kind %d", gate_kind);
    if (gate_kind == kGateElement && (gate_stride % 2 || ((uintptr_t)gate & 3))) return fail("gated_attention_tc: gate rows must start on 4 bytes");
    static bool configured[2] = {false, false};
    if (!configured[softmax ? 1 : 0]) {
        cudaError_t status = softmax ? cudaFuncSetAttribute(gated_attention_tc_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes)
                                     : cudaFuncSetAttribute(gated_attention_tc_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes);
        if (status != cudaSuccess) return fail("gated_attention_tc: cannot reserve %zu bytes of shared memory: %s", kSmemBytes, cudaGetErrorString(status));
        configured[softmax ? 1 : 0] = true;
    }
    const dim3 grid((max_q_len + kQRows - 1) / kQRows, heads, sequences);
    if (softmax)
        MB_LAUNCH("gated_attention_tc", gated_attention_tc_kernel<true>, dim3(grid), dim3(kThreads), kSmemBytes, stream, true, (const bf16*)q,
                  q_stride, (bf16*)out, out_stride, (const bf16*)k_pool, (const bf16*)v_pool, block_table, max_blocks, cu_q, kv_lens, head_bias,
                  (const bf16*)gate, gate_stride, gate_kind, heads, kv_heads, scale, slope_exponent, extras);
    else
        MB_LAUNCH("gated_attention_tc", gated_attention_tc_kernel<false>, dim3(grid), dim3(kThreads), kSmemBytes, stream, true, (const bf16*)q,
                  q_stride, (bf16*)out, out_stride, (const bf16*)k_pool, (const bf16*)v_pool, block_table, max_blocks, cu_q, kv_lens, head_bias,
                  (const bf16*)gate, gate_stride, gate_kind, heads, kv_heads, scale, slope_exponent, extras);
    return check_launch("gated_attention_tc");
}
