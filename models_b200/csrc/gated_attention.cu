// Causal attention over a paged cache for mixers whose weights are not (only) a softmax of scaled dot products,
// in plain float arithmetic; float or bfloat16 storage.
//
//   score(i, j) = scale * q_h(i) . k_c(j) - slope_h * (i - j) + bias_h         c = h / (heads / kv_heads)
//   slope_h = 2^(-slope_exponent * (h + 1) / heads)   (slope_exponent 0: no distance term);  bias absent: 0
//   weight(i, j), j <= i:  softmax over j of score(i, .)     or     sigmoid(score(i, j)), not normalised over j
//   out_h(i) = gate * sum_j weight(i, j) v_c(j)
//   gate: none, sigmoid of one number per (token, head), or sigmoid of one number per output element
//
// Variations of the score (ScoreExtras): a learned factor per head on the scaled product (scale * factor_h * q.k); a
// bound, score <- cap * tanh(score / cap), applied after everything else; a sink, one more term of score 0 that has no
// value in the softmax's denominator, p_j = exp(s_j) / (1 + sum exp(s_j)); and values that were stored rotated by their
// own position (pairs 2m, 2m + 1): the head's sum is then turned back by the query's position before any gate.
// Visibility may be cut into blocks: with `block` n > 0, query i sees key j <= i only if floor(i / n) = floor(j / n)
// (blocks of n positions counted from position 0 of the sequence).
//
// Keys have head_dim coordinates and values value_dim; the value rows may lie in a pool of their own or be the
// first value_dim coordinates of the key rows (a cache that keeps one row per position, read as key and as value).
//
// Cache layout of one layer: k_pool[page][kv_head][page_size][head_dim], v_pool[page][kv_head][page_size][v_width];
// block_table[seq][i] is the page that holds positions [i*page_size, (i+1)*page_size) of that sequence.
//
// Beside the attention: the kernel that normalises query and key heads (RMS norm with a gain shared by the heads),
// scales queries by a temperature that grows with the position, and stores keys and values in the cache; and a
// product with one small matrix per head, out[t, h, :] = W_h in[t, h, :].
#include "common.cuh"

#include <math_constants.h>

MB_DEFINE_LAST_ERROR()

namespace mb {

constexpr int kGateHead = 1, kGateElement = 2;  // gate kinds (0: no gate)

struct ScoreExtras {
    const float* head_scale;  // [heads] factors on the scaled product, or null
    float softcap;            // 0: scores are not bounded
    int sink;                 // != 0: the softmax's denominator has one more term of score 0
    const float* turn_cos;    // [positions][value_dim / 2] with turn_sin: the result's pairs (2m, 2m + 1) are turned by
    const float* turn_sin;    // minus the query's position; null: the result stays as it is
    int block;                // n > 0: a query sees only the keys of its own block of n positions; 0: every earlier key
};

// the first position a query at `pos` sees
__device__ __forceinline__ int lowest_visible(int pos, int block) { return block > 0 ? (pos / block) * block : 0; }

__device__ __forceinline__ float bounded(float z, float cap) { return cap > 0.0f ? cap * tanhf(z / cap) : z; }

// (x, y) of a pair turned by minus the angle whose cosine and sine are c and s.
__device__ __forceinline__ float turned_back(float mine, float partner, bool first_of_pair, float c, float s) {
    return first_of_pair ? mine * c + partner * s : mine * c - partner * s;
}

__device__ __forceinline__ float sigmoid(float v) { return 1.0f / (1.0f + expf(-v)); }

// grid (tokens); block: a multiple of 32 threads; a warp per head.
//   q head (in place): q / rms(q) * q_gain * (1 + temp_coef * ln(floor((p + 1) / temp_every) + 1))
//   k head (into the cache): k / rms(k) * k_gain;  v head (into the cache, if value_dim > 0): as it is.
// rms(x) = sqrt(mean(x^2) + eps).  A null gain means: that side is not normalised.
//
// With a Rotation, query and key heads are first rotated by the token's position over their first `dim` coordinates
// (tables [positions][dim / 2]; pairs (i, i + dim / 2), or (2i, 2i + 1) when `interleaved`), and with `unit` they are then
// divided by their root mean square without any gain; value heads are rotated over their first `value_dim_rotated`
// coordinates by tables of their own on their way into the cache.  Heads of up to 256 coordinates.
struct Rotation {
    const float* cos;
    const float* sin;
    int dim;
    int interleaved;
    int unit;
    const float* value_cos;
    const float* value_sin;
    int value_dim_rotated;
};

// coordinate d of a head rotated by the angle of table row `at` ([dim / 2] cosines and sines)
template <typename T>
__device__ __forceinline__ float rotated_coordinate(const T* __restrict__ src, int d, int dim, int interleaved,
                                                    const float* __restrict__ cos_row, const float* __restrict__ sin_row) {
    const float x = Num<T>::load(src + d);
    if (d >= dim) return x;
    const int half = dim / 2;
    const bool first = interleaved ? (d & 1) == 0 : d < half;
    const int pair = interleaved ? d >> 1 : (d < half ? d : d - half);
    const int other = interleaved ? d ^ 1 : (d < half ? d + half : d - half);
    const float partner = Num<T>::load(src + other);
    return first ? x * cos_row[pair] - partner * sin_row[pair] : x * cos_row[pair] + partner * sin_row[pair];
}

template <typename T>
__global__ void rotate_norm_store_kernel(T* __restrict__ q, int q_stride, const T* __restrict__ k, int k_stride,
                                         const T* __restrict__ v, int v_stride, const int* __restrict__ positions, float eps,
                                         Rotation rotation, T* __restrict__ k_pool, T* __restrict__ v_pool,
                                         const int* __restrict__ slot_mapping, int heads, int kv_heads, int head_dim,
                                         int value_dim, int page_size) {
    grid_launch_dependents();
    grid_dependency_wait();
    constexpr int kPer = 8;
    const int token = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
    const int pos = positions[token];
    const int slot = slot_mapping[token];
    const size_t page = slot >= 0 ? slot / page_size : 0, offset = slot >= 0 ? slot % page_size : 0;
    const float* cos_row = rotation.dim > 0 ? rotation.cos + (size_t)pos * (rotation.dim / 2) : nullptr;
    const float* sin_row = rotation.dim > 0 ? rotation.sin + (size_t)pos * (rotation.dim / 2) : nullptr;
    for (int item = warp; item < heads + kv_heads; item += warps) {
        const bool is_query = item < heads;
        const int head = is_query ? item : item - heads;
        if (!is_query && slot < 0) continue;  // a padding row stores nothing
        T* q_head = q + (size_t)token * q_stride + (size_t)head * head_dim;
        const T* src = is_query ? q_head : k + (size_t)token * k_stride + (size_t)head * head_dim;
        T* dst = is_query ? q_head : k_pool + ((page * kv_heads + head) * page_size + offset) * head_dim;
        float value[kPer];
        float ssq = 0.0f;
#pragma unroll
        for (int i = 0; i < kPer; ++i) {
            const int d = lane + 32 * i;
            value[i] = d < head_dim ? rotated_coordinate<T>(src, d, rotation.dim, rotation.interleaved, cos_row, sin_row) : 0.0f;
            ssq = fmaf(value[i], value[i], ssq);
        }
        __syncwarp();  // a query head is rewritten in place: every lane has read its partners
        const float factor = rotation.unit ? 1.0f / sqrtf(warp_sum(ssq) / (float)head_dim + eps) : 1.0f;
#pragma unroll
        for (int i = 0; i < kPer; ++i) {
            const int d = lane + 32 * i;
            if (d < head_dim) Num<T>::store(dst + d, value[i] * factor);
        }
    }
    if (slot < 0 || value_dim <= 0) return;
    const T* v_row = v + (size_t)token * v_stride;
    const int turned = rotation.value_dim_rotated;
    const float* value_cos = turned > 0 ? rotation.value_cos + (size_t)pos * (turned / 2) : nullptr;
    const float* value_sin = turned > 0 ? rotation.value_sin + (size_t)pos * (turned / 2) : nullptr;
    for (int item = threadIdx.x; item < kv_heads * value_dim; item += blockDim.x) {
        const int head = item / value_dim, d = item % value_dim;
        const float x = rotated_coordinate<T>(v_row + (size_t)head * value_dim, d, turned, rotation.interleaved, value_cos, value_sin);
        Num<T>::store(v_pool + ((page * kv_heads + head) * page_size + offset) * value_dim + d, x);
    }
}

// Two neighbouring elements with one load or store.
template <typename T>
struct Two;
template <>
struct Two<float> {
    static __device__ __forceinline__ float2 load(const float* p) { return *reinterpret_cast<const float2*>(p); }
    static __device__ __forceinline__ void store(float* p, float a, float b) { *reinterpret_cast<float2*>(p) = make_float2(a, b); }
};
template <>
struct Two<__nv_bfloat16> {
    static __device__ __forceinline__ float2 load(const __nv_bfloat16* p) {
        return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p));
    }
    static __device__ __forceinline__ void store(__nv_bfloat16* p, float a, float b) {
        *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(a, b);
    }
};

// The same for pairs (2i, 2i + 1) and even sizes: a lane holds whole pairs, one load and one store per pair, the pair's
// partner never read a second time.  Rows and heads must start on even elements.
template <typename T>
__global__ void rotate_norm_store_pairs_kernel(T* __restrict__ q, int q_stride, const T* __restrict__ k, int k_stride,
                                               const T* __restrict__ v, int v_stride, const int* __restrict__ positions, float eps,
                                               Rotation rotation, T* __restrict__ k_pool, T* __restrict__ v_pool,
                                               const int* __restrict__ slot_mapping, int heads, int kv_heads, int head_dim,
                                               int value_dim, int page_size) {
    grid_launch_dependents();
    grid_dependency_wait();
    constexpr int kPer = 4;  // pairs per lane: heads of up to 256
    const int token = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
    const int pos = positions[token];
    const int slot = slot_mapping[token];
    const size_t page = slot >= 0 ? slot / page_size : 0, offset = slot >= 0 ? slot % page_size : 0;
    const int turning = rotation.dim / 2, pairs = head_dim / 2;
    const float* cos_row = turning > 0 ? rotation.cos + (size_t)pos * turning : nullptr;
    const float* sin_row = turning > 0 ? rotation.sin + (size_t)pos * turning : nullptr;
    for (int item = warp; item < heads + kv_heads; item += warps) {
        const bool is_query = item < heads;
        const int head = is_query ? item : item - heads;
        if (!is_query && slot < 0) continue;  // a padding row stores nothing
        T* q_head = q + (size_t)token * q_stride + (size_t)head * head_dim;
        const T* src = is_query ? q_head : k + (size_t)token * k_stride + (size_t)head * head_dim;
        T* dst = is_query ? q_head : k_pool + ((page * kv_heads + head) * page_size + offset) * head_dim;
        float2 value[kPer];
        float ssq = 0.0f;
#pragma unroll
        for (int i = 0; i < kPer; ++i) {
            const int p = lane + 32 * i;
            value[i] = make_float2(0.0f, 0.0f);
            if (p < pairs) {
                const float2 x = Two<T>::load(src + 2 * p);
                if (p < turning) {
                    const float c = cos_row[p], sn = sin_row[p];
                    value[i] = make_float2(x.x * c - x.y * sn, x.y * c + x.x * sn);
                } else {
                    value[i] = x;
                }
            }
            ssq = fmaf(value[i].x, value[i].x, fmaf(value[i].y, value[i].y, ssq));
        }
        const float factor = rotation.unit ? 1.0f / sqrtf(warp_sum(ssq) / (float)head_dim + eps) : 1.0f;
#pragma unroll
        for (int i = 0; i < kPer; ++i) {
            const int p = lane + 32 * i;
            if (p < pairs) Two<T>::store(dst + 2 * p, value[i].x * factor, value[i].y * factor);
        }
    }
    if (slot < 0 || value_dim <= 0) return;
    const T* v_row = v + (size_t)token * v_stride;
    const int value_turning = rotation.value_dim_rotated / 2, value_pairs = value_dim / 2;
    const float* value_cos = value_turning > 0 ? rotation.value_cos + (size_t)pos * value_turning : nullptr;
    const float* value_sin = value_turning > 0 ? rotation.value_sin + (size_t)pos * value_turning : nullptr;
    for (int item = threadIdx.x; item < kv_heads * value_pairs; item += blockDim.x) {
        const int head = item / value_pairs, p = item % value_pairs;
        float2 x = Two<T>::load(v_row + (size_t)head * value_dim + 2 * p);
        if (p < value_turning) {
            const float c = value_cos[p], sn = value_sin[p];
            x = make_float2(x.x * c - x.y * sn, x.y * c + x.x * sn);
        }
        Two<T>::store(v_pool + ((page * kv_heads + head) * page_size + offset) * value_dim + 2 * p, x.x, x.y);
    }
}

template <typename T>
__global__ void norm_store_kernel(T* __restrict__ q, int q_stride, const T* __restrict__ k, int k_stride,
                                  const T* __restrict__ v, int v_stride, const int* __restrict__ positions,
                                  const float* __restrict__ q_gain, const float* __restrict__ k_gain, float eps,
                                  float temp_coef, int temp_every, T* __restrict__ k_pool, T* __restrict__ v_pool,
                                  const int* __restrict__ slot_mapping, int heads, int kv_heads, int head_dim,
                                  int value_dim, int page_size) {
    grid_launch_dependents();
    grid_dependency_wait();
    const int token = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
    const int pos = positions[token];
    const int slot = slot_mapping[token];
    const size_t page = slot >= 0 ? slot / page_size : 0, offset = slot >= 0 ? slot % page_size : 0;
    float temperature = 1.0f;
    if (temp_coef != 0.0f) temperature = 1.0f + temp_coef * logf((float)((pos + 1) / temp_every) + 1.0f);
    for (int item = warp; item < heads + kv_heads; item += warps) {
        const bool is_query = item < heads;
        const int head = is_query ? item : item - heads;
        const float* gain = is_query ? q_gain : k_gain;
        T* q_head = q + (size_t)token * q_stride + (size_t)head * head_dim;
        const T* src = is_query ? q_head : k + (size_t)token * k_stride + (size_t)head * head_dim;
        if (!is_query && slot < 0) continue;  // a padding row stores nothing
        T* dst = is_query ? q_head : k_pool + ((page * kv_heads + head) * page_size + offset) * head_dim;
        float factor = is_query ? temperature : 1.0f;
        if (gain != nullptr) {
            float ssq = 0.0f;
            for (int d = lane; d < head_dim; d += 32) {
                const float x = Num<T>::load(src + d);
                ssq = fmaf(x, x, ssq);
            }
            ssq = warp_sum(ssq);
            factor *= 1.0f / sqrtf(ssq / (float)head_dim + eps);
        }
        for (int d = lane; d < head_dim; d += 32) {
            float x = Num<T>::load(src + d);
            if (gain != nullptr) x *= gain[d];
            Num<T>::store(dst + d, x * factor);
        }
    }
    if (slot < 0 || value_dim <= 0) return;
    const T* v_row = v + (size_t)token * v_stride;
    for (int item = threadIdx.x; item < kv_heads * value_dim; item += blockDim.x) {
        const int head = item / value_dim, d = item % value_dim;
        v_pool[((page * kv_heads + head) * page_size + offset) * value_dim + d] = v_row[(size_t)head * value_dim + d];
    }
}

// grid (tokens); block 128 or 256.  Query and key projections that are normalised as a WHOLE, all heads at once:
//   q <- (q + q_bias) / rms(q + q_bias) * q_gain over the row of heads * head_dim numbers (rms(x) = sqrt(mean(x^2) + eps);
//   a null gain: that side is not normalised), the same for k over its kv_heads * head_dim numbers; then every head's first
//   `rotation.dim` coordinates are rotated by the token's position (tables as above); q is written back in place, k goes into
//   the cache, and v (+ v_bias) into its pool as it is.  Biases may be null.
// shared: (heads + kv_heads) * head_dim floats (the two rows, so that a pair's partner is read after the norm).
template <typename T>
__global__ void project_norm_rotate_store_kernel(T* __restrict__ q, int q_stride, const T* __restrict__ k, int k_stride,
                                                 const T* __restrict__ v, int v_stride, const float* __restrict__ q_bias,
                                                 const float* __restrict__ k_bias, const float* __restrict__ v_bias,
                                                 const float* __restrict__ q_gain, const float* __restrict__ k_gain, float eps,
                                                 const int* __restrict__ positions, Rotation rotation, T* __restrict__ k_pool,
                                                 T* __restrict__ v_pool, const int* __restrict__ slot_mapping, int heads, int kv_heads,
                                                 int head_dim, int value_dim, int page_size) {
    grid_launch_dependents();
    grid_dependency_wait();
    __shared__ float scratch[32];
    extern __shared__ float both_rows[];
    const int token = blockIdx.x;
    const int q_width = heads * head_dim, k_width = kv_heads * head_dim;
    float* q_row = both_rows;
    float* k_row = both_rows + q_width;
    const int pos = positions[token];
    const int slot = slot_mapping[token];
    const size_t page = slot >= 0 ? slot / page_size : 0, offset = slot >= 0 ? slot % page_size : 0;
    float q_squares = 0.0f, k_squares = 0.0f;
    for (int i = threadIdx.x; i < q_width; i += blockDim.x) {
        const float x = Num<T>::load(q + (size_t)token * q_stride + i) + (q_bias != nullptr ? q_bias[i] : 0.0f);
        q_row[i] = x;
        q_squares = fmaf(x, x, q_squares);
    }
    for (int i = threadIdx.x; i < k_width; i += blockDim.x) {
        const float x = Num<T>::load(k + (size_t)token * k_stride + i) + (k_bias != nullptr ? k_bias[i] : 0.0f);
        k_row[i] = x;
        k_squares = fmaf(x, x, k_squares);
    }
    const float q_factor = q_gain != nullptr ? 1.0f / sqrtf(block_sum(q_squares, scratch) / (float)q_width + eps) : 1.0f;
    const float k_factor = k_gain != nullptr ? 1.0f / sqrtf(block_sum(k_squares, scratch) / (float)k_width + eps) : 1.0f;
    __syncthreads();
    const int turning = rotation.dim, half = rotation.dim / 2;
    const float* cos_row = turning > 0 ? rotation.cos + (size_t)pos * half : nullptr;
    const float* sin_row = turning > 0 ? rotation.sin + (size_t)pos * half : nullptr;
    for (int i = threadIdx.x; i < q_width + k_width; i += blockDim.x) {
        const bool is_query = i < q_width;
        const int at = is_query ? i : i - q_width;
        const int head = at / head_dim, d = at % head_dim;
        const float* row = is_query ? q_row : k_row;
        const float* gain = is_query ? q_gain : k_gain;
        const float factor = is_query ? q_factor : k_factor;
        float x = row[at] * factor * (gain != nullptr ? gain[at] : 1.0f);
        if (d < turning) {
            const bool first = rotation.interleaved ? (d & 1) == 0 : d < half;
            const int pair = rotation.interleaved ? d >> 1 : (d < half ? d : d - half);
            const int other = at - d + (rotation.interleaved ? d ^ 1 : (d < half ? d + half : d - half));
            const float partner = row[other] * factor * (gain != nullptr ? gain[other] : 1.0f);
            x = first ? x * cos_row[pair] - partner * sin_row[pair] : x * cos_row[pair] + partner * sin_row[pair];
        }
        if (is_query)
            Num<T>::store(q + (size_t)token * q_stride + at, x);
        else if (slot >= 0)
            Num<T>::store(k_pool + ((page * kv_heads + head) * page_size + offset) * head_dim + d, x);
    }
    if (slot < 0 || value_dim <= 0) return;
    for (int i = threadIdx.x; i < kv_heads * value_dim; i += blockDim.x) {
        const int head = i / value_dim, d = i % value_dim;
        const float x = Num<T>::load(v + (size_t)token * v_stride + i) + (v_bias != nullptr ? v_bias[i] : 0.0f);
        Num<T>::store(v_pool + ((page * kv_heads + head) * page_size + offset) * value_dim + d, x);
    }
}

template <typename T>
__device__ __forceinline__ float dot_row(const float* __restrict__ q_shared, const T* __restrict__ k_row, int head_dim,
                                         bool vector_ok) {
    float sum = 0.0f;
    if (vector_ok) {
        for (int d = 0; d < head_dim; d += 8) {
            float kv[8];
            load8(k_row + d, kv);
#pragma unroll
            for (int i = 0; i < 8; ++i) sum = fmaf(q_shared[d + i], kv[i], sum);
        }
    } else {
        for (int d = 0; d < head_dim; ++d) sum = fmaf(q_shared[d], Num<T>::load(k_row + d), sum);
    }
    return sum;
}

// One warp per (token, head).  grid (ceil(max_q_len / warps), heads, sequences); block warps * 32.
// kAcc: value coordinates a lane accumulates (value_dim <= 32 * kAcc).  The softmax is the running form: a running
// maximum, partial sums rescaled when it grows.
template <typename T, int kWarps, int kAcc, bool kSoftmax>
__global__ void __launch_bounds__(kWarps * 32)
gated_attention_rows_kernel(const T* __restrict__ q, int q_stride, T* __restrict__ out, int out_stride,
                            const T* __restrict__ k_pool, const T* __restrict__ v_pool, int v_width,
                            const int* __restrict__ block_table, int max_blocks, const int* __restrict__ cu_q,
                            const int* __restrict__ kv_lens, const float* __restrict__ head_bias,
                            const T* __restrict__ gate, int gate_stride, int gate_kind, int heads, int kv_heads,
                            int head_dim, int value_dim, int page_size, float scale, float slope_exponent, ScoreExtras extras) {
    grid_launch_dependents();
    grid_dependency_wait();
    extern __shared__ float q_shared_all[];  // kWarps * head_dim floats
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int seq = blockIdx.z, head = blockIdx.y;
    const int q_begin = cu_q[seq];
    const int q_len = cu_q[seq + 1] - q_begin;
    const int j = blockIdx.x * kWarps + warp;
    if (j >= q_len) return;  // no block-wide barrier below, so a warp may leave alone
    const int row = q_begin + j;
    const int pos = kv_lens[seq] - q_len + j;
    const int kv_head = head / (heads / kv_heads);
    const bool vector_ok = (head_dim % 8) == 0 && (((size_t)k_pool) & (sizeof(T) * 8 - 1)) == 0;
    const float slope = slope_exponent != 0.0f ? exp2f(-slope_exponent * (float)(head + 1) / (float)heads) : 0.0f;
    const float bias = head_bias != nullptr ? head_bias[head] : 0.0f;
    if (extras.head_scale != nullptr) scale *= extras.head_scale[head];

    float* q_shared = q_shared_all + warp * head_dim;
    const T* q_row = q + (size_t)row * q_stride + (size_t)head * head_dim;
    for (int d = lane; d < head_dim; d += 32) q_shared[d] = Num<T>::load(q_row + d);
    __syncwarp();

    float acc[kAcc];
#pragma unroll
    for (int i = 0; i < kAcc; ++i) acc[i] = 0.0f;
    // (a sink is a key of score 0 whose value is zero: it is there before the first chunk)
    float running_max = kSoftmax && extras.sink ? 0.0f : -CUDART_INF_F, running_sum = kSoftmax && extras.sink ? 1.0f : 0.0f;
    const int* table = block_table + (size_t)seq * max_blocks;

    const int lowest = lowest_visible(pos, extras.block);
    for (int chunk = lowest & ~31; chunk <= pos; chunk += 32) {  // (the first chunk holds `lowest`: every chunk has a visible key)
        // page_size is a multiple of 32, so a chunk of 32 positions lies in one page
        const size_t page = table[chunk / page_size];
        const size_t base = (page * kv_heads + kv_head) * page_size + (chunk % page_size);
        const int p = chunk + lane;
        const bool visible = p <= pos && p >= lowest;
        float score = -CUDART_INF_F;
        if (visible)
            score = bounded(dot_row<T>(q_shared, k_pool + (base + lane) * head_dim, head_dim, vector_ok) * scale - slope * (float)(pos - p) + bias,
                            extras.softcap);
        float weight;
        if (kSoftmax) {
            const float new_max = fmaxf(running_max, warp_max(score));  // finite: every chunk holds a visible key
            weight = visible ? expf(score - new_max) : 0.0f;
            const float correction = expf(running_max - new_max);  // exp(-inf) = 0 on the first chunk
            running_sum = running_sum * correction + warp_sum(weight);
            running_max = new_max;
#pragma unroll
            for (int i = 0; i < kAcc; ++i) acc[i] *= correction;
        } else {
            weight = visible ? sigmoid(score) : 0.0f;
        }
        const int last = (pos - chunk < 31) ? pos - chunk : 31;
        for (int jj = max(0, lowest - chunk); jj <= last; ++jj) {  // (keys before the first visible one are not read at all)
            const float w = __shfl_sync(0xffffffffu, weight, jj);
            const T* v_row = v_pool + (base + jj) * v_width;
#pragma unroll
            for (int i = 0; i < kAcc; ++i) {
                const int d = lane + 32 * i;
                if (d < value_dim) acc[i] = fmaf(w, Num<T>::load(v_row + d), acc[i]);
            }
        }
    }
    float factor = kSoftmax ? 1.0f / running_sum : 1.0f;
    if (gate_kind == kGateHead) factor *= sigmoid(Num<T>::load(gate + (size_t)row * gate_stride + head));
    T* out_row = out + (size_t)row * out_stride + (size_t)head * value_dim;
    if (extras.turn_cos != nullptr) {  // (every lane takes part in the exchange; value_dim is even, so a pair is whole)
        const size_t at = (size_t)pos * (value_dim / 2);
#pragma unroll
        for (int i = 0; i < kAcc; ++i) {
            const int d = lane + 32 * i;
            const float partner = __shfl_xor_sync(0xffffffffu, acc[i], 1);
            if (d < value_dim) acc[i] = turned_back(acc[i], partner, (d & 1) == 0, extras.turn_cos[at + d / 2], extras.turn_sin[at + d / 2]);
        }
    }
#pragma unroll
    for (int i = 0; i < kAcc; ++i) {
        const int d = lane + 32 * i;
        if (d < value_dim) {
            float value = acc[i] * factor;
            if (gate_kind == kGateElement)
                value *= sigmoid(Num<T>::load(gate + (size_t)row * gate_stride + (size_t)head * value_dim + d));
            Num<T>::store(out_row + d, value);
        }
    }
}

// ------------------------------------------------------------------------------------------------
// Decoding: one query token per sequence.  A warp per (sequence, head) cannot keep a GPU busy with a handful of
// sequences, and it reads a key/value head once per query head that shares it.  Here the keys of a sequence are cut
// into `splits` runs of `span` pages; a block owns one run of one key/value head and up to kGroup of the query heads
// that share it, so a key or value row is read once for all of them.  Its four warps take the run's chunks of 32 keys
// in turn (a lane a key for the scores, a lane a value coordinate for the sums), then meet in shared memory and write
// one partial result per head: [maximum, sum of weights (softmax) or 1 (sigmoid), value_dim sums]; a run beyond the
// sequence's end writes a sum of 0.  A second kernel adds the runs in their order (rescaled to the common maximum for
// the softmax), applies the gate and stores the token's result: the same bits every time.

// grid (splits, kv_heads * parts, sequences), parts = ceil((heads / kv_heads) / kGroup); block 128.
// shared: q [kGroup][head_dim], then per warp [kGroup][2 + value_dim].
template <typename T, int kGroup, int kAcc, bool kSoftmax>
__global__ void __launch_bounds__(128)
gated_attention_decode_kernel(const T* __restrict__ q, int q_stride, const T* __restrict__ k_pool, const T* __restrict__ v_pool,
                              int v_width, const int* __restrict__ block_table, int max_blocks, const int* __restrict__ cu_q,
                              const int* __restrict__ kv_lens, const float* __restrict__ head_bias, float* __restrict__ partial,
                              int span, int heads, int kv_heads, int head_dim, int value_dim, int page_size, float scale,
                              float slope_exponent, int staged, ScoreExtras extras) {
    grid_launch_dependents();
    grid_dependency_wait();
    extern __shared__ __align__(16) float decode_shared[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int seq = blockIdx.z, split = blockIdx.x, splits = gridDim.x;
    const int group = heads / kv_heads, parts = (group + kGroup - 1) / kGroup;
    const int kv_head = blockIdx.y / parts, part = blockIdx.y % parts;
    const int head0 = kv_head * group + part * kGroup;
    const int count = min(kGroup, group - part * kGroup);
    const int pos = kv_lens[seq] - 1;
    const int lowest = lowest_visible(pos, extras.block);
    const int end = min(pos + 1, (split + 1) * span * page_size);
    const int begin = max(split * span * page_size, lowest & ~31);  // (the chunk of 32 that holds `lowest`: every chunk has a visible key)
    const int stride = 2 + value_dim;
    float* q_shared = decode_shared;
    float* meet = decode_shared + kGroup * head_dim;  // [warp][kGroup][stride]
    // staged: a warp's chunk of 32 key rows (and value rows, where they are rows of their own) comes to shared memory in
    // one batch of 16-byte copies, rows padded by 16 bytes, and is read from there as often as needed: one wait for
    // memory per chunk.  (The rows of a chunk are neighbours in the pool: a chunk lies within a page.)
    const bool own_values = v_pool != k_pool;
    const int k_row_bytes = head_dim * (int)sizeof(T), v_row_bytes = v_width * (int)sizeof(T);
    const int k_pad = k_row_bytes + 16, v_pad = v_row_bytes + 16;
    unsigned char* k_staged = reinterpret_cast<unsigned char*>(meet + 4 * kGroup * stride) + (size_t)warp * 32 * (k_pad + (own_values ? v_pad : 0));
    unsigned char* v_staged = own_values ? k_staged + 32 * k_pad : k_staged;
    if (begin >= end) {  // nothing of the sequence lies in this run (the whole block leaves)
        for (int g = threadIdx.x; g < count; g += blockDim.x) {
            float* dst = partial + (((size_t)seq * heads + head0 + g) * splits + split) * stride;
            dst[0] = -CUDART_INF_F;
            dst[1] = 0.0f;
        }
        return;
    }
    const T* q_row = q + (size_t)cu_q[seq] * q_stride + (size_t)head0 * head_dim;
    for (int i = threadIdx.x; i < count * head_dim; i += blockDim.x) q_shared[i] = Num<T>::load(q_row + i);
    __syncthreads();
    const bool vector_ok = (head_dim % 8) == 0 && (((size_t)k_pool) & (sizeof(T) * 8 - 1)) == 0;
    float slope[kGroup], bias[kGroup], factor_of[kGroup], run_max[kGroup], run_sum[kGroup], acc[kGroup][kAcc];
#pragma unroll
    for (int g = 0; g < kGroup; ++g) {
        slope[g] = slope_exponent != 0.0f ? exp2f(-slope_exponent * (float)(head0 + g + 1) / (float)heads) : 0.0f;
        bias[g] = (head_bias != nullptr && g < count) ? head_bias[head0 + g] : 0.0f;
        factor_of[g] = (extras.head_scale != nullptr && g < count) ? scale * extras.head_scale[head0 + g] : scale;
        run_max[g] = -CUDART_INF_F;
        run_sum[g] = 0.0f;
#pragma unroll
        for (int i = 0; i < kAcc; ++i) acc[g][i] = 0.0f;
    }
    const int* table = block_table + (size_t)seq * max_blocks;
    for (int chunk = begin + warp * 32; chunk < end; chunk += 4 * 32) {
        const size_t page = table[chunk / page_size];
        const size_t base = (page * kv_heads + kv_head) * page_size + (chunk % page_size);
        const int p = chunk + lane;
        const bool visible = p < end && p >= lowest;
        if (staged) {
            __syncwarp();  // the lanes are done with the chunk before
            const unsigned char* k_src = reinterpret_cast<const unsigned char*>(k_pool + base * head_dim);
            const uint32_t k_dst = (uint32_t)__cvta_generic_to_shared(k_staged);
            const int k_pieces = k_row_bytes / 16;
            for (int id = lane; id < 32 * k_pieces; id += 32) {
                const int r = id / k_pieces, piece = id % k_pieces;
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(k_dst + r * k_pad + piece * 16), "l"(k_src + (size_t)r * k_row_bytes + piece * 16));
            }
            if (own_values) {
                const unsigned char* v_src = reinterpret_cast<const unsigned char*>(v_pool + base * v_width);
                const uint32_t v_dst = (uint32_t)__cvta_generic_to_shared(v_staged);
                const int v_pieces = v_row_bytes / 16;
                for (int id = lane; id < 32 * v_pieces; id += 32) {
                    const int r = id / v_pieces, piece = id % v_pieces;
                    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(v_dst + r * v_pad + piece * 16), "l"(v_src + (size_t)r * v_row_bytes + piece * 16));
                }
            }
            asm volatile("cp.async.commit_group;\ncp.async.wait_group 0;\n" ::: "memory");
            __syncwarp();
        }
        float score[kGroup];
#pragma unroll
        for (int g = 0; g < kGroup; ++g) score[g] = 0.0f;
        if (visible) {
            const T* k_row = staged ? reinterpret_cast<const T*>(k_staged + lane * k_pad) : k_pool + (base + lane) * head_dim;
            if (vector_ok) {
#pragma unroll 8
                for (int d = 0; d < head_dim; d += 8) {
                    float kv[8];
                    load8(k_row + d, kv);
#pragma unroll
                    for (int g = 0; g < kGroup; ++g)
                        if (g < count) {
                            const float4 qa = *reinterpret_cast<const float4*>(q_shared + g * head_dim + d);
                            const float4 qb = *reinterpret_cast<const float4*>(q_shared + g * head_dim + d + 4);
                            score[g] = fmaf(qa.x, kv[0], score[g]), score[g] = fmaf(qa.y, kv[1], score[g]);
                            score[g] = fmaf(qa.z, kv[2], score[g]), score[g] = fmaf(qa.w, kv[3], score[g]);
                            score[g] = fmaf(qb.x, kv[4], score[g]), score[g] = fmaf(qb.y, kv[5], score[g]);
                            score[g] = fmaf(qb.z, kv[6], score[g]), score[g] = fmaf(qb.w, kv[7], score[g]);
                        }
                }
            } else {
                for (int d = 0; d < head_dim; ++d) {
                    const float kd = Num<T>::load(k_row + d);
#pragma unroll
                    for (int g = 0; g < kGroup; ++g)
                        if (g < count) score[g] = fmaf(q_shared[g * head_dim + d], kd, score[g]);
                }
            }
        }
        float weight[kGroup];
#pragma unroll
        for (int g = 0; g < kGroup; ++g) {
            const float z = visible ? bounded(score[g] * factor_of[g] - slope[g] * (float)(pos - p) + bias[g], extras.softcap) : -CUDART_INF_F;
            if (kSoftmax) {
                const float new_max = fmaxf(run_max[g], warp_max(z));  // finite: the chunk holds a visible key
                weight[g] = visible ? expf(z - new_max) : 0.0f;
                const float correction = expf(run_max[g] - new_max);
                run_sum[g] = run_sum[g] * correction + warp_sum(weight[g]);
                run_max[g] = new_max;
#pragma unroll
                for (int i = 0; i < kAcc; ++i) acc[g][i] *= correction;
            } else {
                weight[g] = visible ? sigmoid(z) : 0.0f;
            }
        }
        // the values of kAhead keys are asked for before the first is used (a key beyond the run's end has weight 0 and
        // reads the run's last row again)
        constexpr int kAhead = kAcc <= 4 ? 8 : 4;
        const int last = min(31, end - 1 - chunk);
        for (int j0 = max(0, lowest - chunk); j0 <= last; j0 += kAhead) {  // (from the first visible key on)
            float value[kAhead][kAcc];
#pragma unroll
            for (int u = 0; u < kAhead; ++u) {
                const int key = min(j0 + u, last);
                const T* v_row = staged ? reinterpret_cast<const T*>(v_staged + key * (own_values ? v_pad : k_pad)) : v_pool + (base + key) * v_width;
#pragma unroll
                for (int i = 0; i < kAcc; ++i) value[u][i] = lane + 32 * i < value_dim ? Num<T>::load(v_row + lane + 32 * i) : 0.0f;
            }
#pragma unroll
            for (int u = 0; u < kAhead; ++u) {
#pragma unroll
                for (int g = 0; g < kGroup; ++g) {
                    const float w = __shfl_sync(0xffffffffu, weight[g], (j0 + u) & 31);
#pragma unroll
                    for (int i = 0; i < kAcc; ++i) acc[g][i] = fmaf(w, value[u][i], acc[g][i]);
                }
            }
        }
    }
    // the warps meet: every warp leaves its maxima, sums and value sums; the first `count` threads' warps add them in warp order
#pragma unroll
    for (int g = 0; g < kGroup; ++g) {
        if (g < count) {
            float* mine = meet + ((size_t)warp * kGroup + g) * stride;
            if (lane == 0) {
                mine[0] = run_max[g];
                mine[1] = run_sum[g];
            }
#pragma unroll
            for (int i = 0; i < kAcc; ++i)
                if (lane + 32 * i < value_dim) mine[2 + lane + 32 * i] = acc[g][i];
        }
    }
    __syncthreads();
    for (int item = threadIdx.x; item < count * value_dim; item += blockDim.x) {
        const int g = item / value_dim, d = item % value_dim;
        float top = -CUDART_INF_F;
        if (kSoftmax)
            for (int w = 0; w < 4; ++w) top = fmaxf(top, meet[((size_t)w * kGroup + g) * stride]);
        float sum = 0.0f, weights = 0.0f;
        for (int w = 0; w < 4; ++w) {
            const float* theirs = meet + ((size_t)w * kGroup + g) * stride;
            const float factor = kSoftmax ? (theirs[0] == -CUDART_INF_F ? 0.0f : expf(theirs[0] - top)) : 1.0f;
            sum = fmaf(theirs[2 + d], factor, sum);
            weights = fmaf(theirs[1], factor, weights);
        }
        float* dst = partial + (((size_t)seq * heads + head0 + g) * splits + split) * stride;
        dst[2 + d] = sum;
        if (d == 0) {
            dst[0] = top;
            dst[1] = kSoftmax ? weights : 1.0f;
        }
    }
}

// grid (heads, sequences); block: value_dim rounded up to a multiple of 32.
template <typename T, bool kSoftmax>
__global__ void gated_attention_combine_kernel(const float* __restrict__ partial, int splits, T* __restrict__ out, int out_stride,
                                               const int* __restrict__ cu_q, const T* __restrict__ gate, int gate_stride,
                                               int gate_kind, int heads, int value_dim, const int* __restrict__ kv_lens,
                                               ScoreExtras extras) {
    grid_launch_dependents();
    grid_dependency_wait();
    const int head = blockIdx.x, seq = blockIdx.y;
    const bool live = (int)threadIdx.x < value_dim;
    const int d = live ? threadIdx.x : 0;  // (a thread beyond the values follows along for the exchange below and stores nothing)
    const int stride = 2 + value_dim;
    const float* mine = partial + ((size_t)seq * heads + head) * splits * stride;
    const bool sink = kSoftmax && extras.sink;
    float top = sink ? 0.0f : -CUDART_INF_F;
    if (kSoftmax)
        for (int s = 0; s < splits; ++s) top = fmaxf(top, mine[(size_t)s * stride]);
    float sum = 0.0f, weights = sink ? expf(-top) : 0.0f;
    for (int s = 0; s < splits; ++s) {
        const float* run = mine + (size_t)s * stride;
        if (run[1] == 0.0f) continue;  // a run beyond the sequence's end
        const float factor = kSoftmax ? expf(run[0] - top) : 1.0f;
        sum = fmaf(run[2 + d], factor, sum);
        weights = fmaf(run[1], factor, weights);
    }
    float value = kSoftmax ? sum / weights : sum;
    if (extras.turn_cos != nullptr) {
        const size_t at = (size_t)(kv_lens[seq] - 1) * (value_dim / 2) + d / 2;
        const float partner = __shfl_xor_sync(0xffffffffu, value, 1);
        value = turned_back(value, partner, (d & 1) == 0, extras.turn_cos[at], extras.turn_sin[at]);
    }
    if (!live) return;
    const size_t row = cu_q[seq];
    if (gate_kind == kGateHead) value *= sigmoid(Num<T>::load(gate + row * gate_stride + head));
    if (gate_kind == kGateElement) value *= sigmoid(Num<T>::load(gate + row * gate_stride + (size_t)head * value_dim + d));
    Num<T>::store(out + row * out_stride + (size_t)head * value_dim + d, value);
}

// out[t, h * n_out + n] = gate * sum_k in[t, h * n_in + k] * w[(h * n_out + n) * n_in + k]: one small matrix per head,
// rows of n_in weights; gate: sigmoid of gate[t, h] when given.
// Plain arithmetic: grid (ceil(tokens / 16), heads, ceil(n_out / 8)); block 128.  A warp takes 2 of the block's 8
// outputs in turn (few, so that a decode step's handful of tokens still spreads over the multiprocessors and no warp
// waits for memory many times in a row): its lanes walk a weight row together (neighbouring lanes read neighbouring
// weights), each with a sum per token, and the sums meet by shuffles.  shared: 16 * n_in floats.
constexpr int kHeadRows = 16;
constexpr int kHeadOutputs = 8;

template <typename T>
__global__ void head_linear_kernel(const T* __restrict__ in, int in_stride, const T* __restrict__ w, T* __restrict__ out,
                                   int out_stride, const T* __restrict__ gate, int gate_stride, int tokens, int n_in, int n_out) {
    grid_launch_dependents();
    grid_dependency_wait();
    extern __shared__ float rows_shared[];  // [kHeadRows][n_in]
    const int head = blockIdx.y, first = blockIdx.x * kHeadRows;
    const int rows = min(kHeadRows, tokens - first);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int item = threadIdx.x; item < kHeadRows * n_in; item += blockDim.x) {
        const int r = item / n_in, k = item % n_in;
        rows_shared[item] = r < rows ? Num<T>::load(in + (size_t)(first + r) * in_stride + (size_t)head * n_in + k) : 0.0f;
    }
    __syncthreads();
    for (int i = 0; i < kHeadOutputs / 4; ++i) {
        const int n = blockIdx.z * kHeadOutputs + warp * (kHeadOutputs / 4) + i;
        if (n >= n_out) break;
        const T* w_row = w + ((size_t)head * n_out + n) * n_in;
        float acc[kHeadRows];
#pragma unroll
        for (int r = 0; r < kHeadRows; ++r) acc[r] = 0.0f;
        for (int k0 = lane; k0 < n_in; k0 += 32 * 8) {  // eight of the row's weights are asked for before the first is used
            float weight[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) weight[u] = k0 + 32 * u < n_in ? Num<T>::load(w_row + k0 + 32 * u) : 0.0f;
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const int k = min(k0 + 32 * u, n_in - 1);  // (beyond the row the weight is 0)
#pragma unroll
                for (int r = 0; r < kHeadRows; ++r) acc[r] = fmaf(rows_shared[r * n_in + k], weight[u], acc[r]);
            }
        }
        // lane r ends up with token r's sum (every sum is added over the lanes in the same order)
        float mine = 0.0f;
#pragma unroll
        for (int r = 0; r < kHeadRows; ++r) {
            const float total = warp_sum(acc[r]);
            if (lane == r) mine = total;
        }
        if (lane < rows) {
            if (gate != nullptr) mine *= sigmoid(Num<T>::load(gate + (size_t)(first + lane) * gate_stride + head));
            Num<T>::store(out + (size_t)(first + lane) * out_stride + (size_t)head * n_out + n, mine);
        }
    }
}

// The same product on the tensor cores, for bfloat16 steps of many tokens: grid (ceil(tokens / 64), heads); block 128,
// a warp 16 tokens.  The head's 64 x n_in activations and, 64 rows at a time, its weights pass through shared memory
// (cp.async, two stages); m16n8k16 products with float sums.  n_in and n_out are multiples of 16.
namespace tc {

using bf16 = __nv_bfloat16;
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
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

constexpr int kTile = 64;

__global__ void __launch_bounds__(128)
head_linear_tc_kernel(const bf16* __restrict__ in, int in_stride, const bf16* __restrict__ w, bf16* __restrict__ out, int out_stride,
                      const bf16* __restrict__ gate, int gate_stride, int tokens, int n_in, int n_out) {
    grid_launch_dependents();
    grid_dependency_wait();
    extern __shared__ __align__(16) unsigned char tc_smem[];
    const int row_bytes = n_in * 2 + 16, tile_bytes = kTile * row_bytes, pieces = n_in / 8;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, group_id = lane >> 2, tid4 = lane & 3;
    const int head = blockIdx.y, first = blockIdx.x * kTile;
    const int valid = min(kTile, tokens - first);
    const bf16* w_head = w + (size_t)head * n_out * n_in;
    const uint32_t x_tile = smem_u32(tc_smem), w_tiles = x_tile + tile_bytes;
    const int chunks = (n_out + kTile - 1) / kTile;
    auto load_weights = [&](int chunk, int stage) {
        const int rows = min(kTile, n_out - chunk * kTile);  // (a multiple of 16; rows beyond it are never read)
        for (int i = threadIdx.x; i < rows * pieces; i += 128) {
            const int row = i / pieces, piece = i % pieces;
            cp_async16(w_tiles + stage * tile_bytes + row * row_bytes + piece * 16, w_head + (size_t)(chunk * kTile + row) * n_in + piece * 8);
        }
    };
    load_weights(0, 0);
    cp_async_commit();
    for (int i = threadIdx.x; i < kTile * pieces; i += 128) {
        const int row = i / pieces, piece = i % pieces;
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (row < valid) v = *reinterpret_cast<const uint4*>(in + (size_t)(first + row) * in_stride + (size_t)head * n_in + piece * 8);
        *reinterpret_cast<uint4*>(tc_smem + row * row_bytes + piece * 16) = v;
    }
    const uint32_t a_rows = x_tile + (warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * row_bytes + (lane >> 4) * 16;
    float factor[2] = {1.0f, 1.0f};
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int row = warp * 16 + group_id + 8 * r;
        if (gate != nullptr && row < valid) factor[r] = sigmoid(__bfloat162float(gate[(size_t)(first + row) * gate_stride + head]));
    }
    for (int chunk = 0; chunk < chunks; ++chunk) {
        const int stage = chunk & 1;
        if (chunk + 1 < chunks) {
            load_weights(chunk + 1, stage ^ 1);
            cp_async_commit();
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        const int rows = min(kTile, n_out - chunk * kTile);
        const uint32_t w_tile = w_tiles + stage * tile_bytes;
        for (int part = 0; part * 16 < rows; ++part) {
            float s[2][4] = {{0.0f, 0.0f, 0.0f, 0.0f}, {0.0f, 0.0f, 0.0f, 0.0f}};
            const int w_row = part * 16 + (lane & 7) + ((lane >> 4) & 1) * 8;
            for (int ks = 0; ks < n_in / 16; ++ks) {
                uint32_t a[4], b[4];
                ldmatrix_x4(a, a_rows + ks * 32);
                ldmatrix_x4(b, w_tile + w_row * row_bytes + (ks * 2 + ((lane >> 3) & 1)) * 16);
                mma_bf16(s[0], a, b[0], b[1]);
                mma_bf16(s[1], a, b[2], b[3]);
            }
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                const int row = warp * 16 + group_id + 8 * r;
                if (row >= valid) continue;
                bf16* dst = out + (size_t)(first + row) * out_stride + (size_t)head * n_out + chunk * kTile + part * 16 + tid4 * 2;
                *reinterpret_cast<__nv_bfloat162*>(dst) = __floats2bfloat162_rn(s[0][2 * r] * factor[r], s[0][2 * r + 1] * factor[r]);
                *reinterpret_cast<__nv_bfloat162*>(dst + 8) = __floats2bfloat162_rn(s[1][2 * r] * factor[r], s[1][2 * r + 1] * factor[r]);
            }
        }
        __syncthreads();
    }
}

}  // namespace tc

template <typename T>
int launch_norm_store(void* q, int q_stride, const void* k, int k_stride, const void* v, int v_stride, const int* positions,
                      const float* q_gain, const float* k_gain, float eps, float temp_coef, int temp_every, void* k_pool,
                      void* v_pool, const int* slot_mapping, int tokens, int heads, int kv_heads, int head_dim, int value_dim,
                      int page_size, cudaStream_t stream) {
    // a warp per head where a block can have that many (up to 16): a head costs its warp two waits for memory
    const int warps = heads + kv_heads < 4 ? 4 : (heads + kv_heads > 16 ? 16 : heads + kv_heads);
    MB_LAUNCH("norm_store", norm_store_kernel<T>, dim3(tokens), dim3(32 * warps), 0, stream, true, (T*)q, q_stride, (const T*)k,
              k_stride, (const T*)v, v_stride, positions, q_gain, k_gain, eps, temp_coef, temp_every, (T*)k_pool, (T*)v_pool,
              slot_mapping, heads, kv_heads, head_dim, value_dim, page_size);
    return 0;
}

template <typename T>
int launch_rotate_norm_store(void* q, int q_stride, const void* k, int k_stride, const void* v, int v_stride, const int* positions,
                             float eps, Rotation rotation, void* k_pool, void* v_pool, const int* slot_mapping, int tokens, int heads,
                             int kv_heads, int head_dim, int value_dim, int page_size, cudaStream_t stream) {
    const int warps = heads + kv_heads < 4 ? 4 : (heads + kv_heads > 16 ? 16 : heads + kv_heads);
    const bool turns = rotation.dim > 0 || rotation.value_dim_rotated > 0;
    const uintptr_t two = 2 * sizeof(T);
    if ((rotation.interleaved || !turns) && head_dim % 2 == 0 && value_dim % 2 == 0 && q_stride % 2 == 0 && k_stride % 2 == 0 &&
        v_stride % 2 == 0 && !((uintptr_t)q % two) && !((uintptr_t)k % two) && !((uintptr_t)v % two) && !((uintptr_t)k_pool % two) &&
        !((uintptr_t)v_pool % two)) {
        MB_LAUNCH("rotate_norm_store", rotate_norm_store_pairs_kernel<T>, dim3(tokens), dim3(32 * warps), 0, stream, true, (T*)q, q_stride,
                  (const T*)k, k_stride, (const T*)v, v_stride, positions, eps, rotation, (T*)k_pool, (T*)v_pool, slot_mapping, heads,
                  kv_heads, head_dim, value_dim, page_size);
        return 0;
    }
    MB_LAUNCH("rotate_norm_store", rotate_norm_store_kernel<T>, dim3(tokens), dim3(32 * warps), 0, stream, true, (T*)q, q_stride,
              (const T*)k, k_stride, (const T*)v, v_stride, positions, eps, rotation, (T*)k_pool, (T*)v_pool, slot_mapping, heads,
              kv_heads, head_dim, value_dim, page_size);
    return 0;
}

template <typename T, int kAcc, bool kSoftmax>
int launch_rows(const void* q, int q_stride, void* out, int out_stride, const void* k_pool, const void* v_pool, int v_width,
                const int* block_table, int max_blocks, const int* cu_q, const int* kv_lens, const float* head_bias,
                const void* gate, int gate_stride, int gate_kind, int sequences, int max_q_len, int heads, int kv_heads,
                int head_dim, int value_dim, int page_size, float scale, float slope_exponent, ScoreExtras extras, cudaStream_t stream) {
    constexpr int kWarps = 4;
    const dim3 grid((max_q_len + kWarps - 1) / kWarps, heads, sequences);
    const size_t smem = (size_t)kWarps * head_dim * sizeof(float);
    MB_LAUNCH("gated_attention_rows", (gated_attention_rows_kernel<T, kWarps, kAcc, kSoftmax>), dim3(grid), dim3(kWarps * 32), smem,
              stream, true, (const T*)q, q_stride, (T*)out, out_stride, (const T*)k_pool, (const T*)v_pool, v_width, block_table,
              max_blocks, cu_q, kv_lens, head_bias, (const T*)gate, gate_stride, gate_kind, heads, kv_heads, head_dim, value_dim,
              page_size, scale, slope_exponent, extras);
    return 0;
}

template <typename T, bool kSoftmax, typename... Args>
int pick_rows(int value_dim, Args... args) {
    if (value_dim <= 128) return launch_rows<T, 4, kSoftmax>(args...);
    if (value_dim <= 256) return launch_rows<T, 8, kSoftmax>(args...);
    return launch_rows<T, 16, kSoftmax>(args...);
}

}  // namespace mb

using namespace mb;

MB_EXPORT int mb_norm_store(void* q, int q_stride, const void* k, int k_stride, const void* v, int v_stride, int dtype,
                            const int* positions, const float* q_gain, const float* k_gain, float eps, float temp_coef,
                            int temp_every, void* k_pool, void* v_pool, const int* slot_mapping, int tokens, int heads,
                            int kv_heads, int head_dim, int value_dim, int page_size, cudaStream_t stream) {
    if (tokens <= 0) return 0;
    if (head_dim <= 0 || kv_heads <= 0 || heads < 0 || value_dim < 0 || page_size <= 0)
        return fail("norm_store: sizes must be positive (heads %d, kv heads %d, head_dim %d, value_dim %d)", heads, kv_heads, head_dim, value_dim);
    if (temp_every < 1) return fail("norm_store: the temperature's period must be at least 1, got %d", temp_every);
    int status;
    if (dtype == MB_F32)
        status = launch_norm_store<float>(q, q_stride, k, k_stride, v, v_stride, positions, q_gain, k_gain, eps, temp_coef, temp_every,
                                          k_pool, v_pool, slot_mapping, tokens, heads, kv_heads, head_dim, value_dim, page_size, stream);
    else if (dtype == MB_BF16)
        status = launch_norm_store<__nv_bfloat16>(q, q_stride, k, k_stride, v, v_stride, positions, q_gain, k_gain, eps, temp_coef,
                                                  temp_every, k_pool, v_pool, slot_mapping, tokens, heads, kv_heads, head_dim, value_dim,
                                                  page_size, stream);
    else
        return fail("norm_store: unknown dtype code %d", dtype);
    return status ? status : check_launch("norm_store");
}

// Query heads (in place) and key heads (into the cache) rotated by the token's position over their first rotary_dim
// coordinates and then, with unit != 0, divided by their root mean square; value heads rotated over their first
// value_rotary_dim coordinates by tables of their own and stored.  Tables [positions][dim / 2] floats.
MB_EXPORT int mb_rotate_norm_store(void* q, int q_stride, const void* k, int k_stride, const void* v, int v_stride, int dtype,
                                   const int* positions, const float* cos_table, const float* sin_table, int rotary_dim,
                                   int interleaved, int unit, float eps, const float* value_cos, const float* value_sin,
                                   int value_rotary_dim, void* k_pool, void* v_pool, const int* slot_mapping, int tokens, int heads,
                                   int kv_heads, int head_dim, int value_dim, int page_size, cudaStream_t stream) {
    if (tokens <= 0) return 0;
    if (head_dim <= 0 || head_dim > 256 || kv_heads <= 0 || heads < 0 || value_dim < 0 || page_size <= 0)
        return fail("rotate_norm_store: heads %d, kv heads %d, head_dim %d (at most 256), value_dim %d", heads, kv_heads, head_dim, value_dim);
    if (rotary_dim < 0 || rotary_dim % 2 || rotary_dim > head_dim || (rotary_dim > 0 && (cos_table == nullptr || sin_table == nullptr)))
        return fail("rotate_norm_store: rotary_dim %d must be even, at most %d, and come with its tables", rotary_dim, head_dim);
    if (value_rotary_dim < 0 || value_rotary_dim % 2 || value_rotary_dim > value_dim ||
        (value_rotary_dim > 0 && (value_cos == nullptr || value_sin == nullptr)))
        return fail("rotate_norm_store: value_rotary_dim %d must be even, at most %d, and come with its tables", value_rotary_dim, value_dim);
    const Rotation rotation{cos_table, sin_table, rotary_dim, interleaved, unit, value_cos, value_sin, value_rotary_dim};
    int status;
    if (dtype == MB_F32)
        status = launch_rotate_norm_store<float>(q, q_stride, k, k_stride, v, v_stride, positions, eps, rotation, k_pool, v_pool,
                                                 slot_mapping, tokens, heads, kv_heads, head_dim, value_dim, page_size, stream);
    else if (dtype == MB_BF16)
        status = launch_rotate_norm_store<__nv_bfloat16>(q, q_stride, k, k_stride, v, v_stride, positions, eps, rotation, k_pool, v_pool,
                                                         slot_mapping, tokens, heads, kv_heads, head_dim, value_dim, page_size, stream);
    else
        return fail("rotate_norm_store: unknown dtype code %d", dtype);
    return status ? status : check_launch("rotate_norm_store");
}

// q: rows of `heads` heads of head_dim (row stride in elements); out: rows of `heads` heads of value_dim.
// softmax != 0: softmax weights; 0: sigmoid weights.  gate_kind: 0 none, 1 [tokens, heads], 2 [tokens, heads * value_dim].
MB_EXPORT int mb_gated_attention_rows(const void* q, int q_stride, void* out, int out_stride, int dtype, const void* k_pool,
                                      const void* v_pool, int v_width, const int* block_table, int max_blocks, const int* cu_q,
                                      const int* kv_lens, const float* head_bias, const void* gate, int gate_stride, int gate_kind,
                                      int sequences, int max_q_len, int heads, int kv_heads, int head_dim, int value_dim,
                                      int page_size, int softmax, float scale, float slope_exponent, const float* head_scale,
                                      float softcap, int sink, const float* turn_cos, const float* turn_sin, int block, cudaStream_t stream) {
    if (sequences <= 0 || max_q_len <= 0) return 0;
    if ((turn_cos == nullptr) != (turn_sin == nullptr) || (turn_cos != nullptr && value_dim % 2))
        return fail("gated_attention_rows: turning the result back needs both tables and an even value_dim (%d)", value_dim);
    if (softcap < 0.0f || (sink && !softmax)) return fail("gated_attention_rows: softcap %g, a sink without a softmax", softcap);
    const ScoreExtras extras{head_scale, softcap, sink, turn_cos, turn_sin, block};
    if (head_dim <= 0 || head_dim > 2048) return fail("gated_attention_rows: head_dim %d is outside 1..2048", head_dim);
    if (value_dim <= 0 || value_dim > 512 || value_dim > v_width)
        return fail("gated_attention_rows: value_dim %d is outside 1..512 or beyond the value rows of %d", value_dim, v_width);
    if (kv_heads <= 0 || heads % kv_heads) return fail("gated_attention_rows: %d heads are no multiple of %d kv heads", heads, kv_heads);
    if (page_size <= 0 || page_size % 32) return fail("gated_attention_rows: page_size %d must be a multiple of 32", page_size);
    if (sequences > 65535 || heads > 65535) return fail("gated_attention_rows: %d sequences or %d heads exceed the grid limit 65535", sequences, heads);
    if (gate_kind < 0 || gate_kind > 2 || (gate_kind != 0 && gate == nullptr)) return fail("gated_attention_rows: gate kind %d", gate_kind);
    int status;
#define MB_ROWS(T, S)                                                                                                          \
    pick_rows<T, S>(value_dim, q, q_stride, out, out_stride, k_pool, v_pool, v_width, block_table, max_blocks, cu_q, kv_lens,  \
                    head_bias, gate, gate_stride, gate_kind, sequences, max_q_len, heads, kv_heads, head_dim, value_dim,       \
                    page_size, scale, slope_exponent, extras, stream)
    if (dtype == MB_F32)
        status = softmax ? MB_ROWS(float, true) : MB_ROWS(float, false);
    else if (dtype == MB_BF16)
        status = softmax ? MB_ROWS(__nv_bfloat16, true) : MB_ROWS(__nv_bfloat16, false);
    else
        return fail("gated_attention_rows: unknown dtype code %d", dtype);
#undef MB_ROWS
    return status ? status : check_launch("gated_attention_rows");
}

namespace mb {

template <typename T, int kGroup, int kAcc, bool kSoftmax>
int launch_decode(const void* q, int q_stride, void* out, int out_stride, const void* k_pool, const void* v_pool, int v_width,
                  const int* block_table, int max_blocks, const int* cu_q, const int* kv_lens, const float* head_bias,
                  const void* gate, int gate_stride, int gate_kind, int sequences, int heads, int kv_heads, int head_dim,
                  int value_dim, int page_size, float scale, float slope_exponent, int splits, int span, float* partial,
                  ScoreExtras extras, cudaStream_t stream) {
    const int group = heads / kv_heads, parts = (group + kGroup - 1) / kGroup;
    size_t smem = ((size_t)kGroup * head_dim + 4 * (size_t)kGroup * (2 + value_dim)) * sizeof(float);
    // a chunk per warp in shared memory where rows are whole 16-byte pieces and four chunks fit beside the rest
    const size_t k_row = (size_t)head_dim * sizeof(T), v_row = (size_t)v_width * sizeof(T);
    const size_t chunks = 4 * 32 * (k_row + 16 + (v_pool != k_pool ? v_row + 16 : 0));
    const bool staged = k_row % 16 == 0 && v_row % 16 == 0 && !((uintptr_t)k_pool & 15) && !((uintptr_t)v_pool & 15) && smem % 16 == 0 &&
                        smem + chunks <= 160 * 1024;
    if (staged) smem += chunks;
    auto kernel = gated_attention_decode_kernel<T, kGroup, kAcc, kSoftmax>;
    if (smem > 48 * 1024) {
        cudaError_t status = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (status != cudaSuccess) return fail("gated_attention_decode: cannot reserve %zu bytes of shared memory: %s", smem, cudaGetErrorString(status));
    }
    MB_LAUNCH("gated_attention_decode", kernel, dim3(splits, kv_heads * parts, sequences), dim3(128), smem, stream, true, (const T*)q,
              q_stride, (const T*)k_pool, (const T*)v_pool, v_width, block_table, max_blocks, cu_q, kv_lens, head_bias, partial, span,
              heads, kv_heads, head_dim, value_dim, page_size, scale, slope_exponent, staged ? 1 : 0, extras);
    MB_LAUNCH("gated_attention_combine", (gated_attention_combine_kernel<T, kSoftmax>), dim3(heads, sequences),
              dim3((value_dim + 31) / 32 * 32), 0, stream, true, (const float*)partial, splits, (T*)out, out_stride, cu_q,
              (const T*)gate, gate_stride, gate_kind, heads, value_dim, kv_lens, extras);
    return 0;
}

// Eight query heads per block only where that still leaves every multiprocessor several blocks: a warp's work is one long
// chain of dependent steps, so with few sequences more and smaller blocks finish sooner although they read the rows twice.
template <typename T, bool kSoftmax, typename... Args>
int pick_decode(int group, int value_dim, bool many_blocks, Args... args) {
    const bool four = group <= 4 || !many_blocks;
    if (value_dim <= 128) return four ? launch_decode<T, 4, 4, kSoftmax>(args...) : launch_decode<T, 8, 4, kSoftmax>(args...);
    if (value_dim <= 256) return four ? launch_decode<T, 4, 8, kSoftmax>(args...) : launch_decode<T, 8, 8, kSoftmax>(args...);
    return launch_decode<T, 4, 16, kSoftmax>(args...);
}

}  // namespace mb

// Floats of scratch a decode call with `splits` runs needs.
MB_EXPORT size_t mb_gated_attention_decode_scratch_floats(int sequences, int heads, int value_dim, int splits) {
    return (size_t)sequences * heads * splits * (2 + value_dim);
}

// One token per sequence (row cu_q[s] of q and out).  The keys are cut into `splits` runs of `span` pages
// (splits * span * page_size must cover the longest sequence); `partial` holds mb_gated_attention_decode_scratch_floats floats.
MB_EXPORT int mb_gated_attention_decode(const void* q, int q_stride, void* out, int out_stride, int dtype, const void* k_pool,
                                        const void* v_pool, int v_width, const int* block_table, int max_blocks, const int* cu_q,
                                        const int* kv_lens, const float* head_bias, const void* gate, int gate_stride, int gate_kind,
                                        int sequences, int heads, int kv_heads, int head_dim, int value_dim, int page_size,
                                        int softmax, float scale, float slope_exponent, int splits, int span, float* partial,
                                        const float* head_scale, float softcap, int sink, const float* turn_cos,
                                        const float* turn_sin, int block, cudaStream_t stream) {
    if (sequences <= 0) return 0;
    if ((turn_cos == nullptr) != (turn_sin == nullptr) || (turn_cos != nullptr && value_dim % 2))
        return fail("gated_attention_decode: turning the result back needs both tables and an even value_dim (%d)", value_dim);
    if (softcap < 0.0f || (sink && !softmax)) return fail("gated_attention_decode: softcap %g, a sink without a softmax", softcap);
    const ScoreExtras extras{head_scale, softcap, sink, turn_cos, turn_sin, block};
    if (head_dim <= 0 || head_dim > 2048) return fail("gated_attention_decode: head_dim %d is outside 1..2048", head_dim);
    if (value_dim <= 0 || value_dim > 512 || value_dim > v_width)
        return fail("gated_attention_decode: value_dim %d is outside 1..512 or beyond the value rows of %d", value_dim, v_width);
    if (kv_heads <= 0 || heads % kv_heads) return fail("gated_attention_decode: %d heads are no multiple of %d kv heads", heads, kv_heads);
    if (page_size <= 0 || page_size % 32) return fail("gated_attention_decode: page_size %d must be a multiple of 32", page_size);
    if (splits < 1 || span < 1 || splits > 65535) return fail("gated_attention_decode: %d runs of %d pages", splits, span);
    if (sequences > 65535 || heads > 65535) return fail("gated_attention_decode: %d sequences or %d heads exceed the grid limit 65535", sequences, heads);
    if (gate_kind < 0 || gate_kind > 2 || (gate_kind != 0 && gate == nullptr)) return fail("gated_attention_decode: gate kind %d", gate_kind);
    if (partial == nullptr) return fail("gated_attention_decode: no scratch memory");
    const bool many_blocks = (long long)sequences * kv_heads * ((heads / kv_heads + 7) / 8) * splits >= 4 * 148;
    int status;
#define MB_DECODE(T, S)                                                                                                          \
    mb::pick_decode<T, S>(heads / kv_heads, value_dim, many_blocks, q, q_stride, out, out_stride, k_pool, v_pool, v_width, block_table,       \
                          max_blocks, cu_q, kv_lens, head_bias, gate, gate_stride, gate_kind, sequences, heads, kv_heads, head_dim, \
                          value_dim, page_size, scale, slope_exponent, splits, span, partial, extras, stream)
    if (dtype == MB_F32)
        status = softmax ? MB_DECODE(float, true) : MB_DECODE(float, false);
    else if (dtype == MB_BF16)
        status = softmax ? MB_DECODE(__nv_bfloat16, true) : MB_DECODE(__nv_bfloat16, false);
    else
        return fail("gated_attention_decode: unknown dtype code %d", dtype);
#undef MB_DECODE
    return status ? status : check_launch("gated_attention_decode");
}

// tensor_cores != 0 asks for the tensor-core form where it applies (bfloat16, n_in and n_out multiples of 16, rows that
// start on 16 bytes (in) and 4 bytes (out), at least 16 tokens).
MB_EXPORT int mb_head_linear(const void* in, int in_stride, const void* w, void* out, int out_stride, int dtype, const void* gate,
                             int gate_stride, int tokens, int heads, int n_in, int n_out, int tensor_cores, cudaStream_t stream) {
    if (tokens <= 0 || heads <= 0) return 0;
    if (n_in <= 0 || n_out <= 0) return fail("head_linear: sizes must be positive, got %d -> %d", n_in, n_out);
    if (heads > 65535) return fail("head_linear: %d heads exceed the grid limit 65535", heads);
    if (tensor_cores && dtype == MB_BF16 && tokens >= 16 && n_in % 16 == 0 && n_out % 16 == 0 && n_in <= 512 && in_stride % 8 == 0 &&
        out_stride % 2 == 0 && !((uintptr_t)in & 15) && !((uintptr_t)w & 15) && !((uintptr_t)out & 3)) {
        const size_t smem = 3 * (size_t)tc::kTile * (n_in * 2 + 16);
        static int reserved = 0;
        if ((int)smem > reserved) {
            cudaError_t status = cudaFuncSetAttribute(tc::head_linear_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (status != cudaSuccess) return fail("head_linear: cannot reserve %zu bytes of shared memory: %s", smem, cudaGetErrorString(status));
            reserved = (int)smem;
        }
        MB_LAUNCH("head_linear_tc", tc::head_linear_tc_kernel, dim3((tokens + tc::kTile - 1) / tc::kTile, heads), dim3(128), smem, stream, true,
                  (const __nv_bfloat16*)in, in_stride, (const __nv_bfloat16*)w, (__nv_bfloat16*)out, out_stride, (const __nv_bfloat16*)gate,
                  gate_stride, tokens, n_in, n_out);
        return check_launch("head_linear_tc");
    }
    const size_t smem = (size_t)kHeadRows * n_in * sizeof(float);
    if (smem > 200 * 1024) return fail("head_linear: %d inputs per head exceed a block's shared memory", n_in);
    const dim3 grid((tokens + kHeadRows - 1) / kHeadRows, heads, (n_out + kHeadOutputs - 1) / kHeadOutputs);
    if (dtype == MB_F32) {
        if (smem > 48 * 1024) cudaFuncSetAttribute(head_linear_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        MB_LAUNCH("head_linear", head_linear_kernel<float>, dim3(grid), dim3(128), smem, stream, true, (const float*)in, in_stride,
                  (const float*)w, (float*)out, out_stride, (const float*)gate, gate_stride, tokens, n_in, n_out);
    } else if (dtype == MB_BF16) {
        if (smem > 48 * 1024) cudaFuncSetAttribute(head_linear_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        MB_LAUNCH("head_linear", head_linear_kernel<__nv_bfloat16>, dim3(grid), dim3(128), smem, stream, true, (const __nv_bfloat16*)in,
                  in_stride, (const __nv_bfloat16*)w, (__nv_bfloat16*)out, out_stride, (const __nv_bfloat16*)gate, gate_stride, tokens,
                  n_in, n_out);
    } else {
        return fail("head_linear: unknown dtype code %d", dtype);
    }
    return check_launch("head_linear");
}

// q (in place), k and v rows of one storage type (row strides in elements); biases and gains float or null; cos/sin tables
// [positions][rotary_dim / 2] (rotary_dim 0: no rotation).
MB_EXPORT int mb_project_norm_rotate_store(void* q, int q_stride, const void* k, int k_stride, const void* v, int v_stride, int dtype,
                                           const float* q_bias, const float* k_bias, const float* v_bias, const float* q_gain,
                                           const float* k_gain, float eps, const int* positions, const float* cos, const float* sin,
                                           int rotary_dim, int interleaved, void* k_pool, void* v_pool, const int* slot_mapping,
                                           int tokens, int heads, int kv_heads, int head_dim, int value_dim, int page_size,
                                           cudaStream_t stream) {
    if (tokens <= 0) return 0;
    if (rotary_dim < 0 || rotary_dim % 2 || rotary_dim > head_dim) return fail("project_norm_rotate_store: rotary_dim %d of heads of %d", rotary_dim, head_dim);
    const size_t smem = sizeof(float) * (size_t)(heads + kv_heads) * head_dim;
    if (smem > 40 * 1024) return fail("project_norm_rotate_store: rows of %d numbers exceed the 10240 a block keeps", (heads + kv_heads) * head_dim);
    const Rotation rotation{cos, sin, rotary_dim, interleaved, 0, nullptr, nullptr, 0};
    const int threads = (heads + kv_heads) * head_dim >= 1024 ? 256 : 128;
    if (dtype == MB_F32)
        MB_LAUNCH("project_norm_rotate_store", project_norm_rotate_store_kernel<float>, dim3(tokens), dim3(threads), smem, stream, true,
                  (float*)q, q_stride, (const float*)k, k_stride, (const float*)v, v_stride, q_bias, k_bias, v_bias, q_gain, k_gain, eps,
                  positions, rotation, (float*)k_pool, (float*)v_pool, slot_mapping, heads, kv_heads, head_dim, value_dim, page_size);
    else if (dtype == MB_BF16)
        MB_LAUNCH("project_norm_rotate_store", project_norm_rotate_store_kernel<__nv_bfloat16>, dim3(tokens), dim3(threads), smem, stream,
                  true, (__nv_bfloat16*)q, q_stride, (const __nv_bfloat16*)k, k_stride, (const __nv_bfloat16*)v, v_stride, q_bias, k_bias,
                  v_bias, q_gain, k_gain, eps, positions, rotation, (__nv_bfloat16*)k_pool, (__nv_bfloat16*)v_pool, slot_mapping, heads,
                  kv_heads, head_dim, value_dim, page_size);
    else
        return fail("project_norm_rotate_store: unknown dtype code %d", dtype);
    return check_launch("project_norm_rotate_store");
}
