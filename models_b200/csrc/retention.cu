// Retention: linear attention with a fixed decay per head and a float state per sequence and head, over the new
// tokens of ragged sequences.
//
//   q_t, k_t: rotated over their first rotary_dim coordinates (split-half pairs, angles from float tables by the
//             token's position), k_t then multiplied by key_scale
//   S_t = decay_h S_(t-1) + k_t v_t^T          S [head_dim, value_dim], float, one per (sequence, head), kept between steps
//   o_t = S_t^T q_t
//   y_t = out_scale * o_t / sqrt(mean(o_t^2) + eps) * silu(g_t)          (the mean over the head's value_dim numbers)
//
// Variations: `input_act` >= 0 applies that activation of the activation table to q, k and v as they are read (before
// any rotation); with `raw_out` the kernel stops after o_t and writes out_scale * o_t as floats (no norm, no gate): what
// comes after it is then another kernel's, for instance one norm over all heads (group_norm_gate below).
//
// q, k, v, g are projections of the token (storage type, float or bfloat16); everything after them is float.
//
// A block owns one (sequence, head): a thread per value coordinate j keeps column j of S in shared memory
// ([head_dim][value_dim], so that neighbouring threads touch neighbouring words) and walks the sequence's new tokens
// in order.  The state is read from the state area when the block starts and written back when it ends.
//
// The recurrence is linear in S, so a step of many tokens is cut into runs of `run_length` consecutive tokens that are
// walked at the same time, in three kernels: every run first walks its tokens from a zero state and leaves what it
// adds, B_r = sum_j decay^(n_r - 1 - j) k_j v_j^T, in scratch memory; then, element by element, the runs' starting
// states follow from the stored state in run order, S_(r+1) = decay^(n_r) S_r + B_r (the last one is the sequence's new
// state); then every run walks its tokens again from its starting state and writes the results.
#include "common.cuh"

MB_DEFINE_LAST_ERROR()

namespace mb {

constexpr int kWhole = 0;      // one run: from the stored state, results written, the state stored
constexpr int kSummarise = 1;  // a run from a zero state, no results: what it adds goes to scratch [run]
constexpr int kEmit = 2;       // a run from its starting state in scratch [run], results written
constexpr int kTokens = 8;     // tokens of a group: their inputs are fetched together, their norms taken together

// Bytes of a group's raw rows, rounded up to 16.
__host__ __device__ inline size_t raw_row_bytes(int row, size_t element) { return ((size_t)kTokens * row * element + 15) / 16 * 16; }

// grid (heads, sequences, runs); block: value_dim rounded up to a multiple of 32 (at most 1024; 256 with kDim > 0).
// kDim > 0: head_dim is kDim and a thread keeps its column of S in registers (a column in shared memory costs two
// shared-memory accesses per product, which is what bounds the kernel then); kDim 0: any head_dim, columns in shared memory.
// A run is walked in groups of kTokens tokens: the group's rotated queries, scaled rotated keys, values and gates are
// brought to shared memory as floats by all threads at once (one wait for memory per group instead of one per token,
// into the buffer the group before does not use), the threads walk the group's tokens, leave their o in shared memory,
// and the warps then take the tokens' root mean squares and write the results.
// shared: 2 buffers [kTokens][2 head_dim + 2 value_dim], o [kTokens][value_dim], and with kDim 0 S [head_dim * value_dim].
// scratch: [sequence][head][run][head_dim * value_dim] floats.
template <typename T, int kMode, int kDim>
__global__ void __launch_bounds__(kDim > 0 ? 256 : 1024)
retention_scan_kernel(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v, const T* __restrict__ g,
                      int in_stride, const int* __restrict__ positions, const float* __restrict__ cos_table,
                      const float* __restrict__ sin_table, int rotary_dim, const float* __restrict__ decay, float key_scale,
                      float eps, float* __restrict__ state, const int* __restrict__ slots, const int* __restrict__ cu_q,
                      int heads, int head_dim, int value_dim, T* __restrict__ out, int out_stride, float out_scale,
                      int run_length, float* __restrict__ scratch, int async_ok, int input_act, float* __restrict__ raw_out,
                      int raw_stride) {
    grid_launch_dependents();
    grid_dependency_wait();
    extern __shared__ __align__(16) float shared[];
    const int head = blockIdx.x, seq = blockIdx.y, run = blockIdx.z;
    const int sequence_first = cu_q[seq];
    const int sequence_count = cu_q[seq + 1] - sequence_first;
    const int first = sequence_first + run * run_length;
    const int count = kMode == kWhole ? sequence_count : min(run_length, sequence_count - run * run_length);
    if (count <= 0) return;  // the whole block leaves
    const int row = 2 * head_dim + 2 * value_dim;  // a token's staged floats: q, k, v, g
    float* staged = shared;
    float* results = staged + 2 * kTokens * row;
    // raw: the next group's rows as they lie in memory (storage type) and its rows of the rotation tables, copied by
    // cp.async while the group before is walked
    const int half_early = rotary_dim / 2;
    T* raw = reinterpret_cast<T*>(results + kTokens * value_dim);
    float* raw_cos = reinterpret_cast<float*>(reinterpret_cast<unsigned char*>(raw) + raw_row_bytes(row, sizeof(T)));
    float* raw_sin = raw_cos + kTokens * half_early;
    float* S = raw_sin + kTokens * half_early + ((4 - (2 * kTokens * half_early) % 4) % 4);  // (kDim 0 only)
    float column_kept[kDim > 0 ? kDim : 1];
    const int j = threadIdx.x;
    const bool live = j < value_dim;
    const int half = rotary_dim / 2;
    const float a = decay[head];
    const bool no_gate = kMode == kSummarise || raw_out != nullptr;
    float* stored = kMode == kWhole ? state + ((size_t)slots[seq] * heads + head) * head_dim * value_dim
                                    : scratch + (((size_t)seq * heads + head) * gridDim.z + run) * head_dim * value_dim;
    if (kDim > 0) {
#pragma unroll
        for (int d = 0; d < kDim; ++d) column_kept[d] = (kMode == kSummarise || !live) ? 0.0f : stored[(size_t)d * value_dim + j];
    } else if (live) {
        for (int d = 0; d < head_dim; ++d) S[d * value_dim + j] = kMode == kSummarise ? 0.0f : stored[(size_t)d * value_dim + j];
    }

    // The tokens t0 .. t0 + n - 1 of the run into buffer b.  A thread takes coordinate c of the staged row [q | k | v | g]
    // for all tokens of the group: what c is (which tensor, rotated or not, its pair) is worked out once, and the
    // group's loads are all asked for before the first is stored.  A sequence's new tokens stand at consecutive
    // positions, so a token's position follows from the first one's without a load per token.
    const int position0 = positions[sequence_first] + run * run_length;
    auto stage = [&](int t0, int n, int b) {
        for (int c = threadIdx.x; c < row; c += blockDim.x) {
            const bool is_qk = c < 2 * head_dim;
            const bool is_key = is_qk && c >= head_dim;
            const bool is_gate = !is_qk && c >= 2 * head_dim + value_dim;
            if ((kMode == kSummarise && is_qk && !is_key) || (no_gate && is_gate)) continue;  // no results: no queries, no gates
            const int d = is_qk ? (is_key ? c - head_dim : c) : c - 2 * head_dim - (is_gate ? value_dim : 0);
            const bool activated = input_act >= 0 && !is_gate;
            const T* source = (is_qk ? (is_key ? k : q) + (size_t)head * head_dim : (is_gate ? g : v) + (size_t)head * value_dim)
                              + (size_t)(first + t0) * in_stride;
            const bool rotated = is_qk && d < rotary_dim;
            const int pair = d < half ? d : d - half;
            const int other = d < half ? d + half : d - half;
            const float sign = d < half ? -1.0f : 1.0f;
            float value[kTokens];
#pragma unroll
            for (int u = 0; u < kTokens; ++u) {
                value[u] = 0.0f;
                if (u < n) {
                    const T* x = source + (size_t)u * in_stride;
                    value[u] = Num<T>::load(x + d);
                    if (activated) value[u] = gate_activation(input_act, value[u]);
                    if (rotated) {
                        const size_t at = (size_t)(position0 + t0 + u) * half + pair;
                        float partner = Num<T>::load(x + other);
                        if (activated) partner = gate_activation(input_act, partner);
                        value[u] = value[u] * cos_table[at] + sign * partner * sin_table[at];
                    }
                }
            }
            const float factor = is_key ? key_scale : 1.0f;
#pragma unroll
            for (int u = 0; u < kTokens; ++u)
                if (u < n) staged[(b * kTokens + u) * row + c] = value[u] * factor;
        }
    };

    // The same in two steps, for rows that cp.async can copy (async_ok: every row and table row starts on 16 bytes and is
    // whole 16-byte pieces): `issue` starts the copies of a group's raw rows and returns; `convert`, after they have
    // arrived, turns them into the staged floats from shared memory.  The copies fly while the group before is walked.
    auto issue = [&](int t0, int n) {
        const int piece = 16 / (int)sizeof(T);
        const int qk_pieces = head_dim / piece, v_pieces = value_dim / piece, token_pieces = 2 * qk_pieces + 2 * v_pieces;
        const uint32_t raw_at = (uint32_t)__cvta_generic_to_shared(raw);
        for (int id = threadIdx.x; id < n * token_pieces; id += blockDim.x) {
            const int u = id / token_pieces, p = id % token_pieces;
            const T* source;
            int c;  // the piece's first coordinate in the staged row
            if (p < 2 * qk_pieces) {
                const bool is_key = p >= qk_pieces;
                if (kMode == kSummarise && !is_key) continue;
                const int d = (is_key ? p - qk_pieces : p) * piece;
                source = (is_key ? k : q) + (size_t)head * head_dim + d;
                c = (is_key ? head_dim : 0) + d;
            } else {
                const int pv = p - 2 * qk_pieces;
                const bool is_gate = pv >= v_pieces;
                if (no_gate && is_gate) continue;
                const int d = (is_gate ? pv - v_pieces : pv) * piece;
                source = (is_gate ? g : v) + (size_t)head * value_dim + d;
                c = 2 * head_dim + (is_gate ? value_dim : 0) + d;
            }
            source += (size_t)(first + t0 + u) * in_stride;
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(raw_at + (uint32_t)((u * row + c) * sizeof(T))), "l"(source));
        }
        if (rotary_dim > 0) {
            const int table_pieces = half / 4;
            const uint32_t cos_at = (uint32_t)__cvta_generic_to_shared(raw_cos), sin_at = (uint32_t)__cvta_generic_to_shared(raw_sin);
            for (int id = threadIdx.x; id < n * 2 * table_pieces; id += blockDim.x) {
                const int u = id / (2 * table_pieces), p = id % (2 * table_pieces);
                const bool is_sin = p >= table_pieces;
                const int at = (is_sin ? p - table_pieces : p) * 4;
                const float* source = (is_sin ? sin_table : cos_table) + (size_t)(position0 + t0 + u) * half + at;
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"((is_sin ? sin_at : cos_at) + (uint32_t)((u * half + at) * 4)), "l"(source));
            }
        }
        asm volatile("cp.async.commit_group;\n" ::);
    };
    auto convert = [&](int n, int b) {
        for (int c = threadIdx.x; c < row; c += blockDim.x) {
            const bool is_qk = c < 2 * head_dim;
            const bool is_key = is_qk && c >= head_dim;
            const bool is_gate = !is_qk && c >= 2 * head_dim + value_dim;
            if ((kMode == kSummarise && is_qk && !is_key) || (no_gate && is_gate)) continue;
            const int d = is_qk ? (is_key ? c - head_dim : c) : 0;
            const bool activated = input_act >= 0 && !is_gate;
            const bool rotated = is_qk && d < rotary_dim;
            const int pair = d < half ? d : d - half;
            const int other = c + (d < half ? half : -half);
            const float sign = d < half ? -1.0f : 1.0f;
            const float factor = is_key ? key_scale : 1.0f;
#pragma unroll
            for (int u = 0; u < kTokens; ++u) {
                if (u >= n) break;
                float value = Num<T>::load(raw + u * row + c);
                if (activated) value = gate_activation(input_act, value);
                if (rotated) {
                    float partner = Num<T>::load(raw + u * row + other);
                    if (activated) partner = gate_activation(input_act, partner);
                    value = value * raw_cos[u * half + pair] + sign * partner * raw_sin[u * half + pair];
                }
                staged[(b * kTokens + u) * row + c] = value * factor;
            }
        }
    };

    if (async_ok) {
        issue(0, min(kTokens, count));
        asm volatile("cp.async.wait_group 0;\n" ::: "memory");
        __syncthreads();
        convert(min(kTokens, count), 0);
    } else {
        stage(0, min(kTokens, count), 0);
    }
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
    for (int t0 = 0; t0 < count; t0 += kTokens) {
        const int b = (t0 / kTokens) & 1;
        const int n = min(kTokens, count - t0);
        const float* group = staged + b * kTokens * row;
        const bool more = t0 + kTokens < count;
        const int n_next = more ? min(kTokens, count - t0 - kTokens) : 0;
        if (async_ok && more) issue(t0 + kTokens, n_next);  // under way while this group is walked
        if (live) {
#pragma unroll
            for (int u = 0; u < kTokens; ++u) {
                if (u >= n) break;
                const float* qs = group + u * row;
                const float* ks = qs + head_dim;
                const float vj = qs[2 * head_dim + j];
                float o = 0.0f;
                if (kDim > 0) {
                    float part[4] = {0.0f, 0.0f, 0.0f, 0.0f};  // four chains of sums instead of one of kDim
#pragma unroll
                    for (int d = 0; d < kDim; d += 4) {
                        const float4 k4 = *reinterpret_cast<const float4*>(ks + d);
                        column_kept[d] = fmaf(a, column_kept[d], k4.x * vj);
                        column_kept[d + 1] = fmaf(a, column_kept[d + 1], k4.y * vj);
                        column_kept[d + 2] = fmaf(a, column_kept[d + 2], k4.z * vj);
                        column_kept[d + 3] = fmaf(a, column_kept[d + 3], k4.w * vj);
                        if (kMode != kSummarise) {
                            const float4 q4 = *reinterpret_cast<const float4*>(qs + d);
                            part[0] = fmaf(column_kept[d], q4.x, part[0]);
                            part[1] = fmaf(column_kept[d + 1], q4.y, part[1]);
                            part[2] = fmaf(column_kept[d + 2], q4.z, part[2]);
                            part[3] = fmaf(column_kept[d + 3], q4.w, part[3]);
                        }
                    }
                    o = (part[0] + part[1]) + (part[2] + part[3]);
                } else {
                    float* column = S + j;
#pragma unroll 4
                    for (int d = 0; d < head_dim; ++d) {
                        const float s = fmaf(a, column[d * value_dim], ks[d] * vj);
                        column[d * value_dim] = s;
                        if (kMode != kSummarise) o = fmaf(s, qs[d], o);
                    }
                }
                if (kMode != kSummarise) results[u * value_dim + j] = o;
            }
        }
        if (!async_ok && more) stage(t0 + kTokens, n_next, b ^ 1);  // the other buffer
        if (async_ok) asm volatile("cp.async.wait_group 0;\n" ::: "memory");
        __syncthreads();  // the group's o and the next group's inputs (staged, or raw) are in shared memory
        if (async_ok && more) convert(n_next, b ^ 1);
        if (kMode == kSummarise && async_ok) __syncthreads();  // the next group's staged floats, before they are read
        if (kMode != kSummarise) {
            for (int u = warp; u < n; u += warps) {  // a warp per token: root mean square of the head's o, gate, store
                const float* o_row = results + u * value_dim;
                if (raw_out != nullptr) {  // the caller norms and gates
                    float* raw_row = raw_out + (size_t)(first + t0 + u) * raw_stride + (size_t)head * value_dim;
                    for (int d = lane; d < value_dim; d += 32) raw_row[d] = o_row[d] * out_scale;
                    continue;
                }
                const float* gate_row = group + u * row + 2 * head_dim + value_dim;
                float ssq = 0.0f;
                for (int d = lane; d < value_dim; d += 32) ssq = fmaf(o_row[d], o_row[d], ssq);
                const float inverse = out_scale / sqrtf(warp_sum(ssq) / (float)value_dim + eps);
                T* out_row = out + (size_t)(first + t0 + u) * out_stride + (size_t)head * value_dim;
                for (int d = lane; d < value_dim; d += 32) {
                    const float gate = gate_row[d];
                    Num<T>::store(out_row + d, o_row[d] * inverse * (gate / (1.0f + expf(-gate))));
                }
            }
            __syncthreads();  // the next group writes its o over these
        }
    }
    if (live && kMode != kEmit) {
        if (kDim > 0) {
#pragma unroll
            for (int d = 0; d < kDim; ++d) stored[(size_t)d * value_dim + j] = column_kept[d];
        } else {
            for (int d = 0; d < head_dim; ++d) stored[(size_t)d * value_dim + j] = S[d * value_dim + j];
        }
    }
}

// The runs' starting states, element by element in run order: scratch [run] holds what run `run` adds and receives the
// state the run starts from; the state after the last run goes back to the state area.
// grid (ceil(head_dim * value_dim / 256), heads, sequences); block 256.
__global__ void retention_prefix_kernel(float* __restrict__ scratch, float* __restrict__ state, const int* __restrict__ slots,
                                        const int* __restrict__ cu_q, const float* __restrict__ decay, int heads, int elements,
                                        int runs, int run_length) {
    grid_launch_dependents();
    grid_dependency_wait();
    const int head = blockIdx.y, seq = blockIdx.z;
    const int e = blockIdx.x * blockDim.x + threadIdx.x;
    const int count = cu_q[seq + 1] - cu_q[seq];
    if (e >= elements || count <= 0) return;
    float* stored = state + ((size_t)slots[seq] * heads + head) * elements + e;
    float* mine = scratch + ((size_t)seq * heads + head) * runs * elements + e;
    const float a = decay[head];
    const float whole_run = powf(a, (float)run_length);
    float s = *stored;
    const int used = (count + run_length - 1) / run_length;
    for (int run0 = 0; run0 < used; run0 += 8) {  // eight runs' additions are asked for before the first start is stored
        float added[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) added[u] = run0 + u < used ? mine[(size_t)(run0 + u) * elements] : 0.0f;
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const int run = run0 + u;
            if (run < used) {
                const int n = min(run_length, count - run * run_length);
                mine[(size_t)run * elements] = s;
                s = fmaf(n == run_length ? whole_run : powf(a, (float)n), s, added[u]);
            }
        }
    }
    *stored = s;
}

// y[t] = raw[t] / sqrt(mean(raw[t]^2) + eps) * gain * act(gate[t]) over a whole row (all heads together);
// gate_sigmoid != 0: sigmoid, else silu.  grid (rows); block 256.
template <typename T>
__global__ void __launch_bounds__(256)
group_norm_gate_kernel(const float* __restrict__ raw, int raw_stride, const float* __restrict__ gain, const T* __restrict__ gate,
                       int gate_stride, T* __restrict__ out, int out_stride, int width, float eps, int gate_sigmoid) {
    grid_launch_dependents();
    grid_dependency_wait();
    __shared__ float scratch[32];
    const size_t row = blockIdx.x;
    const float* mine = raw + row * raw_stride;
    float ssq = 0.0f;
    for (int c = threadIdx.x; c < width; c += blockDim.x) ssq = fmaf(mine[c], mine[c], ssq);
    const float inverse = 1.0f / sqrtf(block_sum(ssq, scratch) / (float)width + eps);
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        const float g = Num<T>::load(gate + row * gate_stride + c);
        const float s = 1.0f / (1.0f + expf(-g));
        Num<T>::store(out + row * out_stride + c, mine[c] * inverse * gain[c] * (gate_sigmoid ? s : g * s));
    }
}

}  // namespace mb

using namespace mb;

MB_EXPORT int mb_group_norm_gate(const float* raw, int raw_stride, const float* gain, const void* gate, int gate_stride, void* out,
                                 int out_stride, int dtype, int rows, int width, float eps, int gate_sigmoid, cudaStream_t stream) {
    if (rows <= 0 || width <= 0) return 0;
    if (dtype == MB_F32)
        MB_LAUNCH("group_norm_gate", group_norm_gate_kernel<float>, dim3(rows), dim3(256), 0, stream, true, raw, raw_stride, gain,
                  (const float*)gate, gate_stride, (float*)out, out_stride, width, eps, gate_sigmoid);
    else if (dtype == MB_BF16)
        MB_LAUNCH("group_norm_gate", group_norm_gate_kernel<__nv_bfloat16>, dim3(rows), dim3(256), 0, stream, true, raw, raw_stride, gain,
                  (const __nv_bfloat16*)gate, gate_stride, (__nv_bfloat16*)out, out_stride, width, eps, gate_sigmoid);
    else
        return fail("group_norm_gate: unknown dtype code %d", dtype);
    return 0;
}

// q, k: [tokens, >= heads * head_dim]; v, g: [tokens, >= heads * value_dim]; all four column slices of one tensor
// (one row stride).  state: float [slots, heads, head_dim, value_dim]; slots[sequence] picks the row.
// rotary_dim 0: no rotation (the tables may then be null).
MB_EXPORT size_t mb_retention_scratch_floats(int sequences, int heads, int head_dim, int value_dim, int max_q_len, int run_length) {
    if (run_length <= 0 || max_q_len <= run_length) return 0;
    return (size_t)sequences * heads * ((max_q_len + run_length - 1) / run_length) * head_dim * value_dim;
}

namespace mb {

template <typename T, int kDim>
int launch_retention(const void* q, const void* k, const void* v, const void* g, int in_stride, const int* positions,
                     const float* cos_table, const float* sin_table, int rotary_dim, const float* decay, float key_scale, float eps,
                     float* state, const int* slots, const int* cu_q, int sequences, int heads, int head_dim, int value_dim, void* out,
                     int out_stride, float out_scale, int max_q_len, int run_length, float* scratch, int input_act, float* raw_out,
                     int raw_stride, cudaStream_t stream, size_t smem) {
    const dim3 block((value_dim + 31) / 32 * 32);
    const int runs = (run_length > 0 && max_q_len > run_length) ? (max_q_len + run_length - 1) / run_length : 1;
    // rows that cp.async can copy: every row and table row starts on 16 bytes and is whole 16-byte pieces
    const size_t element = sizeof(T);
    const int async_ok = ((size_t)in_stride * element) % 16 == 0 && ((size_t)head_dim * element) % 16 == 0 &&
                         ((size_t)value_dim * element) % 16 == 0 && !((uintptr_t)q & 15) && !((uintptr_t)k & 15) && !((uintptr_t)v & 15) &&
                         !((uintptr_t)g & 15) &&
                         (rotary_dim == 0 || ((rotary_dim / 2) % 4 == 0 && !((uintptr_t)cos_table & 15) && !((uintptr_t)sin_table & 15)));
    if (smem > 48 * 1024) {
        cudaFuncSetAttribute(retention_scan_kernel<T, kWhole, kDim>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        cudaFuncSetAttribute(retention_scan_kernel<T, kSummarise, kDim>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        cudaFuncSetAttribute(retention_scan_kernel<T, kEmit, kDim>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    }
#define MB_SCAN(MODE, RUNS)                                                                                                      \
    MB_LAUNCH("retention_scan", (retention_scan_kernel<T, MODE, kDim>), dim3(heads, sequences, RUNS), dim3(block), smem, stream, true,  \
              (const T*)q, (const T*)k, (const T*)v, (const T*)g, in_stride, positions, cos_table, sin_table, rotary_dim, decay,  \
              key_scale, eps, state, slots, cu_q, heads, head_dim, value_dim, (T*)out, out_stride, out_scale, run_length, scratch, \
              async_ok, input_act, raw_out, raw_stride)
    if (runs == 1) {
        MB_SCAN(kWhole, 1);
        return 0;
    }
    const int elements = head_dim * value_dim;
    MB_SCAN(kSummarise, runs);
    MB_LAUNCH("retention_prefix", retention_prefix_kernel, dim3((elements + 255) / 256, heads, sequences), dim3(256), 0, stream, true,
              scratch, state, slots, cu_q, decay, heads, elements, runs, run_length);
    MB_SCAN(kEmit, runs);
#undef MB_SCAN
    return 0;
}

// Columns of S in registers where head_dim is one of the sizes compiled for and a block of value_dim threads may have them.
template <typename T, typename... Args>
int pick_retention(int head_dim, int value_dim, size_t smem_shared, size_t smem_kept, Args... args) {
    if (value_dim <= 256 && value_dim % 2 == 0) {  // (even: a token's staged floats then start on 16 bytes)
        if (head_dim == 16) return launch_retention<T, 16>(args..., smem_kept);
        if (head_dim == 32) return launch_retention<T, 32>(args..., smem_kept);
        if (head_dim == 64) return launch_retention<T, 64>(args..., smem_kept);
        if (head_dim == 128) return launch_retention<T, 128>(args..., smem_kept);
    }
    return launch_retention<T, 0>(args..., smem_shared);
}

}  // namespace mb

// q, k: [tokens, >= heads * head_dim]; v, g: [tokens, >= heads * value_dim]; all four column slices of one tensor
// (one row stride).  state: float [slots, heads, head_dim, value_dim]; slots[sequence] picks the row.
// rotary_dim 0: no rotation (the tables may then be null).  With max_q_len > run_length > 0 the sequences are walked in
// runs of run_length tokens at once, and scratch must hold mb_retention_scratch_floats floats.
// input_act: -1, or a code of the activation table applied to q, k, v.  raw_out non-null: out_scale * o_t goes there as
// floats ([tokens][raw_stride], heads side by side) and nothing else is written; g and out may then be null.
MB_EXPORT int mb_retention_scan(const void* q, const void* k, const void* v, const void* g, int in_stride, int dtype,
                                const int* positions, const float* cos_table, const float* sin_table, int rotary_dim,
                                const float* decay, float key_scale, float eps, float* state, const int* slots, const int* cu_q,
                                int sequences, int heads, int head_dim, int value_dim, void* out, int out_stride, float out_scale,
                                int max_q_len, int run_length, float* scratch, int input_act, float* raw_out, int raw_stride,
                                cudaStream_t stream) {
    if (sequences <= 0 || heads <= 0) return 0;
    if (input_act >= MB_ACT_COUNT) return fail("retention_scan: unknown activation code %d", input_act);
    if (head_dim <= 0 || value_dim <= 0 || value_dim > 1024) return fail("retention_scan: head_dim %d, value_dim %d (at most 1024)", head_dim, value_dim);
    if (rotary_dim < 0 || rotary_dim % 2 || rotary_dim > head_dim) return fail("retention_scan: rotary_dim %d must be even and at most %d", rotary_dim, head_dim);
    if (rotary_dim > 0 && (cos_table == nullptr || sin_table == nullptr)) return fail("retention_scan: rotation needs its tables");
    if (sequences > 65535) return fail("retention_scan: %d sequences exceed the grid limit 65535", sequences);
    if (run_length > 0 && max_q_len > run_length && scratch == nullptr) return fail("retention_scan: runs need scratch memory");
    if (run_length > 0 && (max_q_len + run_length - 1) / run_length > 65535) return fail("retention_scan: too many runs");
    const size_t element = dtype == MB_F32 ? 4 : 2;
    const size_t smem_kept = ((size_t)2 * kTokens * (2 * head_dim + 2 * value_dim) + (size_t)kTokens * value_dim) * sizeof(float) +
                             raw_row_bytes(2 * head_dim + 2 * value_dim, element) + ((size_t)2 * kTokens * (rotary_dim / 2) + 4) * sizeof(float);
    const size_t smem = smem_kept + (size_t)head_dim * value_dim * sizeof(float);
    const bool kept = value_dim <= 256 && value_dim % 2 == 0 && (head_dim == 16 || head_dim == 32 || head_dim == 64 || head_dim == 128);
    if (!kept && smem > 227 * 1024) return fail("retention_scan: a state of %d x %d floats exceeds a block's shared memory", head_dim, value_dim);
    int status;
    if (dtype == MB_F32)
        status = pick_retention<float>(head_dim, value_dim, smem, smem_kept, q, k, v, g, in_stride, positions, cos_table, sin_table,
                                       rotary_dim, decay, key_scale, eps, state, slots, cu_q, sequences, heads, head_dim, value_dim, out,
                                       out_stride, out_scale, max_q_len, run_length, scratch, input_act, raw_out, raw_stride, stream);
    else if (dtype == MB_BF16)
        status = pick_retention<__nv_bfloat16>(head_dim, value_dim, smem, smem_kept, q, k, v, g, in_stride, positions, cos_table, sin_table,
                                               rotary_dim, decay, key_scale, eps, state, slots, cu_q, sequences, heads, head_dim, value_dim,
                                               out, out_stride, out_scale, max_q_len, run_length, scratch, input_act, raw_out, raw_stride,
                                               stream);
    else
        return fail("retention_scan: unknown dtype code %d", dtype);
    return status ? status : check_launch("retention_scan");
}
