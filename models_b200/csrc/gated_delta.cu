// Short causal convolutions over time, and the gated delta rule; ragged sequences, per-sequence state kept in float.
//
// Short convolution, per channel c with `taps` weights w[c][0 .. taps - 1] whose LAST one meets the current token:
//   x_t = in_t (+ in_bias);   out_t = act(sum_i w[c][taps - 1 - i] x_(t - i) (+ out_bias)),   x = 0 before the sequence starts.
// The last taps - 1 inputs x of every sequence are part of its state: `tail` [taps - 1][channels], oldest first.  The kernel
// computes the new tokens' results from the stored tail and the step's inputs and stores the new tail.
//
// Gated delta rule, per head h with its float state S [dim][vdim] (query/key head c = h / (heads / kv_heads)):
//   q_t, k_t: the convolved rows made unit vectors, x / sqrt(sum x^2 + unit_eps); q_t also times dim^(-1/2)
//   beta_t = sigmoid(b_t);   g_t = exp(decay_h * softplus(a_t + dt_bias_h))          (decay_h = -exp(A_log_h), a number <= 0)
//   S <- g_t S;   u = beta_t (v_t - S^T k_t);   S <- S + k_t u^T;   o_t = S^T q_t    (the read-out sees the token's own write)
//   out_t = out_scale * o_t / rms(o_t) * gain * silu(gate_t),   rms over the head's vdim numbers, gain [vdim] shared by the heads
// Everything after the projections is float arithmetic.  A block owns 32 columns of one (sequence, head); a column of S lives
// in the registers of four neighbouring lanes, and the tokens pass in groups of 16 whose rows arrive in shared memory while the
// group before is walked; norm, gain and gate follow in a kernel with a warp per (token, head).
#include "common.cuh"

MB_DEFINE_LAST_ERROR()

namespace mb {

constexpr int kMaxTaps = 8;
constexpr int kConvTokens = 16;  // tokens a thread of the convolution walks
constexpr int kGroup = 16;       // tokens of a group of the delta rule's walk

__device__ __forceinline__ float sigmoid(float v) { return 1.0f / (1.0f + expf(-v)); }
__device__ __forceinline__ float softplus(float v) { return fmaxf(v, 0.0f) + log1pf(expf(-fabsf(v))); }

// grid (ceil(channels / 128), ceil(max_q_len / kConvTokens), sequences); block 128.  The thread that walks a sequence's first
// tokens is the only one that reads the stored tail of its channel; with `store_tail` it also stores the new one (the last
// taps - 1 inputs, from the step's tokens and, where the step brought fewer, from the old tail), so that no second kernel is
// needed.  `split` (or null): the results also as two bfloat16 numbers each, rounding and rest, block by block of `per`
// channels: [token][block][rounding of the block's channels | rests], what a tensor-core product with float-like accuracy reads.
template <typename T>
__global__ void __launch_bounds__(128)
short_conv_kernel(const T* __restrict__ in, int in_stride, const float* __restrict__ in_bias, const float* __restrict__ weights,
                  const float* __restrict__ out_bias, int activation, float* __restrict__ out, int out_stride,
                  float* __restrict__ state, size_t state_stride, const int* __restrict__ slots, const int* __restrict__ cu_q,
                  int channels, int taps, int store_tail, __nv_bfloat16* __restrict__ split, int per) {
    grid_launch_dependents();
    grid_dependency_wait();
    const int c = blockIdx.x * blockDim.x + threadIdx.x, seq = blockIdx.z;
    const int first = cu_q[seq], count = cu_q[seq + 1] - first;
    const int j0 = blockIdx.y * kConvTokens, j1 = min(j0 + kConvTokens, count);
    if (c >= channels || j0 >= count) return;
    float* tail = state + (size_t)slots[seq] * state_stride;
    const float bias_in = in_bias != nullptr ? in_bias[c] : 0.0f, bias_out = out_bias != nullptr ? out_bias[c] : 0.0f;
    float w[kMaxTaps], x[kMaxTaps];  // w[i] meets the input i tokens back; x[i] is that input
#pragma unroll
    for (int i = 0; i < kMaxTaps; ++i) {
        w[i] = i < taps ? weights[(size_t)c * taps + (taps - 1 - i)] : 0.0f;
        x[i] = 0.0f;
        if (i >= 1 && i < taps) {
            const int j = j0 - i;
            x[i] = j >= 0 ? Num<T>::load(in + (size_t)(first + j) * in_stride + c) + bias_in : tail[(size_t)(taps - 1 + j) * channels + c];
        }
    }
    if (store_tail && j0 == 0) {
#pragma unroll
        for (int i = 0; i < kMaxTaps; ++i)
            if (i < taps - 1) {  // tail row i is the input of token count - (taps - 1) + i; a negative token is an old row, held in x
                const int j = count - (taps - 1) + i;
                float kept = 0.0f;
#pragma unroll
                for (int back = 1; back < kMaxTaps; ++back)
                    if (back == -j) kept = x[back];
                tail[(size_t)i * channels + c] = j >= 0 ? Num<T>::load(in + (size_t)(first + j) * in_stride + c) + bias_in : kept;
            }
    }
    for (int j = j0; j < j1; ++j) {
        x[0] = Num<T>::load(in + (size_t)(first + j) * in_stride + c) + bias_in;
        float sum = 0.0f;
#pragma unroll
        for (int i = kMaxTaps - 1; i >= 0; --i) sum = fmaf(w[i], x[i], sum);  // oldest input first
        sum += bias_out;
        if (activation == 1) sum = sum * sigmoid(sum);
        out[(size_t)(first + j) * out_stride + c] = sum;
        if (split != nullptr) {
            const __nv_bfloat16 rounding = __float2bfloat16_rn(sum);
            __nv_bfloat16* row = split + (size_t)(first + j) * 2 * channels + (size_t)(c / per) * 2 * per + c % per;
            row[0] = rounding;
            row[per] = __float2bfloat16_rn(sum - __bfloat162float(rounding));
        }
#pragma unroll
        for (int i = kMaxTaps - 1; i >= 1; --i) x[i] = x[i - 1];
    }
}

struct DeltaShape {
    int heads, kv_heads, dim, vdim;
    int q_at, k_at, v_at;  // first columns of the convolved rows' q, k and v parts
};

__device__ __forceinline__ void copy_float_async(float* dst, const float* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src));
}

// grid (ceil(tokens * 2 * kv_heads / 4)); block 128: a warp per (token, query or key head).  In place on the convolved rows:
// x <- factor * x / sqrt(sum x^2 + unit_eps), factor dim^(-1/2) for query heads and 1 for key heads.
__global__ void __launch_bounds__(128)
unit_heads_kernel(float* __restrict__ conv, int conv_stride, int items, float unit_eps, DeltaShape shape) {
    grid_launch_dependents();
    grid_dependency_wait();
    const int item = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (item >= items) return;
    const int per_token = 2 * shape.kv_heads;
    const size_t token = item / per_token;
    const int which = item % per_token;
    const bool is_query = which < shape.kv_heads;
    float* x = conv + token * conv_stride + (is_query ? shape.q_at + which * shape.dim : shape.k_at + (which - shape.kv_heads) * shape.dim);
    float squares = 0.0f;
    for (int d = lane; d < shape.dim; d += 32) squares = fmaf(x[d], x[d], squares);
    const float factor = (is_query ? 1.0f / sqrtf((float)shape.dim) : 1.0f) / sqrtf(warp_sum(squares) + unit_eps);
    for (int d = lane; d < shape.dim; d += 32) x[d] *= factor;
}

// The walk.  grid (heads, sequences, ceil(vdim / 32)); block 128: a block owns 32 columns of a head's state (columns do not
// depend on one another, so a head spreads over several multiprocessors: the work of a token, 3 dim vdim multiply-adds, would
// otherwise bound the walk by what ONE multiprocessor issues).  A column is shared out over kSplit neighbouring lanes, each with
// the kPer coordinates d = part * kPer + i in registers (dim <= kSplit * kPer); the two sums over d of a token meet by shuffles.
// (With one sequence the walk is a chain of dependent instructions: eight lanes a column give a multiprocessor's schedulers two
// warps each and a thread a short chain; a profile of four lanes a column showed one warp per scheduler issuing every fifth cycle.)
// Only S^T k stands on the path from one token to the next; the read-out S^T q overlaps with the next token's.  Tokens pass in
// groups of kGroup whose convolved rows arrive in shared memory by cp.async while the group before is walked (two buffers); beta
// and g of the next group are fetched a group ahead as well.  q and k arrive as unit vectors (unit_heads_kernel ran before).
// The raw read-outs o go to `raw` (float [tokens][heads * vdim]);
// norm, gain and gate follow in a kernel of their own, which needs every column of a head.
// shared: 2 x (q [kGroup][kD], k [kGroup][kD], v [kGroup][32]), 2 x (beta, g) [kGroup]; kD = kSplit * kPer.
constexpr int kColumns = 32;  // columns of a block

template <typename T, int kPer, int kSplit>
__global__ void __launch_bounds__(kColumns * kSplit)
gated_delta_walk_kernel(const float* __restrict__ conv, int conv_stride, const T* __restrict__ a_in, const T* __restrict__ b_in,
                        int in_stride, const float* __restrict__ decay, const float* __restrict__ dt_bias,
                        float* __restrict__ state, size_t state_stride, const int* __restrict__ slots, const int* __restrict__ cu_q,
                        float* __restrict__ raw, DeltaShape shape) {
    grid_launch_dependents();
    grid_dependency_wait();
    constexpr int kD = kSplit * kPer;
    extern __shared__ __align__(16) float delta_shared[];
    const int head = blockIdx.x, seq = blockIdx.y;
    const int first = cu_q[seq], count = cu_q[seq + 1] - first;
    if (count <= 0) return;
    const int dim = shape.dim, vdim = shape.vdim;
    const int qk_head = head / (shape.heads / shape.kv_heads);
    const int tid = threadIdx.x;
    const int col0 = blockIdx.z * kColumns, local = tid / kSplit, col = col0 + local, part = tid % kSplit;
    const int here = min(kColumns, vdim - col0);  // columns of this block
    constexpr int buffer_floats = kGroup * (2 * kD + kColumns);
    float* gates = delta_shared + 2 * buffer_floats;  // [2][beta kGroup | g kGroup]
    const bool live = col < vdim;
    float* stored = state + (size_t)slots[seq] * state_stride + (size_t)head * dim * vdim;
    float s[kPer];
#pragma unroll
    for (int i = 0; i < kPer; ++i) {
        const int d = part * kPer + i;
        s[i] = (live && d < dim) ? stored[(size_t)d * vdim + col] : 0.0f;
    }
    const float head_decay = decay[head], head_dt = dt_bias[head];
    const int groups = (count + kGroup - 1) / kGroup;
    const size_t raw_stride = (size_t)shape.heads * vdim;

    auto fetch = [&](int group) {  // the convolved rows of a group into its buffer (the coordinates beyond dim stay zero)
        float* q_s = delta_shared + (group & 1) * buffer_floats;
        float* k_s = q_s + kGroup * kD;
        float* v_s = k_s + kGroup * kD;
        const int t0 = group * kGroup, n = min(kGroup, count - t0);
        for (int i = tid; i < n * dim; i += blockDim.x) {
            const int u = i / dim, d = i % dim;
            const float* row = conv + (size_t)(first + t0 + u) * conv_stride;
            copy_float_async(q_s + u * kD + d, row + shape.q_at + qk_head * dim + d);
            copy_float_async(k_s + u * kD + d, row + shape.k_at + qk_head * dim + d);
        }
        for (int i = tid; i < n * here; i += blockDim.x) {
            const int u = i / here, j = i % here;
            copy_float_async(v_s + u * kColumns + j, conv + (size_t)(first + t0 + u) * conv_stride + shape.v_at + head * vdim + col0 + j);
        }
        asm volatile("cp.async.commit_group;\n" ::);
    };
    for (int i = tid; i < 2 * buffer_floats; i += blockDim.x) delta_shared[i] = 0.0f;  // (zeros beyond dim and beyond the columns, once)
    __syncthreads();
    fetch(0);
    if (tid < min(kGroup, count)) {
        const size_t at = (size_t)(first + tid) * in_stride + head;
        gates[tid] = sigmoid(Num<T>::load(b_in + at));
        gates[kGroup + tid] = expf(head_decay * softplus(Num<T>::load(a_in + at) + head_dt));
    }
    for (int group = 0; group < groups; ++group) {
        const int t0 = group * kGroup, n = min(kGroup, count - t0);
        float* q_s = delta_shared + (group & 1) * buffer_floats;
        float* k_s = q_s + kGroup * kD;
        const float* v_s = k_s + kGroup * kD;
        const float* beta_s = gates + (group & 1) * 2 * kGroup;
        const float* g_s = beta_s + kGroup;
        float a_next = 0.0f, b_next = 0.0f;
        const bool more = group + 1 < groups;
        const bool mine_next = more && tid < min(kGroup, count - t0 - kGroup);
        if (more) {
            fetch(group + 1);  // (its buffer was last read a group ago, before that group's closing barrier)
            if (mine_next) {
                const size_t at = (size_t)(first + t0 + kGroup + tid) * in_stride + head;
                a_next = Num<T>::load(a_in + at);
                b_next = Num<T>::load(b_in + at);
            }
            asm volatile("cp.async.wait_group 1;\n" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;\n" ::: "memory");
        }
        __syncthreads();
        float* raw_at = raw + (size_t)(first + t0) * raw_stride + (size_t)head * vdim + col;
        // a token's k, q, v, beta and g are taken from shared memory while the token before is worked on (their addresses do not
        // depend on the recurrence), so the chain from token to token holds arithmetic and shuffles only
        float k[kPer], q[kPer], k_ahead[kPer], q_ahead[kPer];
        float v = 0.0f, beta = 0.0f, g = 0.0f, v_ahead, beta_ahead, g_ahead;
        auto take = [&](int u, float (&kk)[kPer], float (&qq)[kPer], float& vv, float& bb, float& gg) {
            const float4* k4 = reinterpret_cast<const float4*>(k_s + u * kD + part * kPer);
            const float4* q4 = reinterpret_cast<const float4*>(q_s + u * kD + part * kPer);
#pragma unroll
            for (int i = 0; i < kPer; i += 4) {
                const float4 a = k4[i / 4], b = q4[i / 4];
                kk[i] = a.x, kk[i + 1] = a.y, kk[i + 2] = a.z, kk[i + 3] = a.w;
                qq[i] = b.x, qq[i + 1] = b.y, qq[i + 2] = b.z, qq[i + 3] = b.w;
            }
            vv = v_s[u * kColumns + local];
            bb = beta_s[u];
            gg = g_s[u];
        };
        take(0, k, q, v, beta, g);
        // In program order (a warp issues in order): the partial sum S^T k of token u was taken while token u - 1 was finished;
        // its shuffles run side by side with those of token u - 1's read-out; then the write, the update of S, and in ONE loop the
        // read-out's partial sum and the next token's S^T k.
        float seen = 0.0f, o_before = 0.0f;
#pragma unroll
        for (int i = 0; i < kPer; ++i) seen = fmaf(s[i], k[i], seen);
#pragma unroll  // (all of a group's tokens spelled out: the rows' places in shared memory are constants and no register is copied)
        for (int u = 0; u < kGroup; ++u) {
            if (u >= n) break;
            take(u + 1 < kGroup ? u + 1 : u, k_ahead, q_ahead, v_ahead, beta_ahead, g_ahead);  // (a row beyond the group's tokens holds finite leftovers)
            float decayed[kPer];
#pragma unroll
            for (int i = 0; i < kPer; ++i) decayed[i] = g * s[i];
#pragma unroll
            for (int offset = 1; offset < kSplit; offset <<= 1) {
                seen += __shfl_xor_sync(0xffffffffu, seen, offset);
                o_before += __shfl_xor_sync(0xffffffffu, o_before, offset);
            }
            if (u > 0 && live && part == 0) raw_at[(size_t)(u - 1) * raw_stride] = o_before;
            const float write = beta * (v - g * seen);  // (S^T k of the decayed state is g times the old one's)
            float o0 = 0.0f, o1 = 0.0f, next0 = 0.0f, next1 = 0.0f;
#pragma unroll
            for (int i = 0; i < kPer; i += 2) {
                s[i] = fmaf(k[i], write, decayed[i]);
                s[i + 1] = fmaf(k[i + 1], write, decayed[i + 1]);
                o0 = fmaf(s[i], q[i], o0);
                next0 = fmaf(s[i], k_ahead[i], next0);
                o1 = fmaf(s[i + 1], q[i + 1], o1);
                next1 = fmaf(s[i + 1], k_ahead[i + 1], next1);
            }
            o_before = o0 + o1;
            seen = next0 + next1;
#pragma unroll
            for (int i = 0; i < kPer; ++i) k[i] = k_ahead[i], q[i] = q_ahead[i];
            v = v_ahead, beta = beta_ahead, g = g_ahead;
        }
#pragma unroll
        for (int offset = 1; offset < kSplit; offset <<= 1) o_before += __shfl_xor_sync(0xffffffffu, o_before, offset);
        if (live && part == 0) raw_at[(size_t)(n - 1) * raw_stride] = o_before;
        if (mine_next) {
            float* next = gates + ((group + 1) & 1) * 2 * kGroup;
            next[tid] = sigmoid(b_next);
            next[kGroup + tid] = expf(head_decay * softplus(a_next + head_dt));
        }
        __syncthreads();  // the group's buffer may be filled again
    }
    if (live) {
#pragma unroll
        for (int i = 0; i < kPer; ++i) {
            const int d = part * kPer + i;
            if (d < dim) stored[(size_t)d * vdim + col] = s[i];
        }
    }
}

// grid (ceil(tokens * heads / 4)); block 128: a warp per (token, head).  out = out_scale * o / rms(o) * gain * silu(gate).
template <typename T>
__global__ void __launch_bounds__(128)
head_norm_gate_kernel(const float* __restrict__ raw, const T* __restrict__ gate_in, int gate_stride, const float* __restrict__ gain,
                      float eps, T* __restrict__ out, int out_stride, float out_scale, int items, int heads, int vdim) {
    grid_launch_dependents();
    grid_dependency_wait();
    const int item = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (item >= items) return;
    const size_t token = item / heads;
    const int head = item % heads;
    const float* o = raw + token * heads * vdim + (size_t)head * vdim;
    float squares = 0.0f;
    for (int j = lane; j < vdim; j += 32) squares = fmaf(o[j], o[j], squares);
    const float inv = out_scale / sqrtf(warp_sum(squares) / (float)vdim + eps);
    for (int j = lane; j < vdim; j += 32) {
        const float z = Num<T>::load(gate_in + token * gate_stride + (size_t)head * vdim + j);
        Num<T>::store(out + token * out_stride + (size_t)head * vdim + j, o[j] * inv * gain[j] * (z * sigmoid(z)));
    }
}

template <typename T, int kPer, int kSplit>
int launch_delta_walk(const float* conv, int conv_stride, const void* a_in, const void* b_in, int in_stride, const float* decay,
                      const float* dt_bias, float* state, size_t state_stride, const int* slots, const int* cu_q,
                      int sequences, float* raw, DeltaShape shape, cudaStream_t stream) {
    const size_t smem = sizeof(float) * (2 * (size_t)kGroup * (2 * kSplit * kPer + kColumns) + 4 * kGroup);
    if (smem > 48 * 1024) {
        cudaError_t status = cudaFuncSetAttribute(gated_delta_walk_kernel<T, kPer, kSplit>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (status != cudaSuccess) return fail("gated_delta_scan: cannot reserve %zu bytes of shared memory: %s", smem, cudaGetErrorString(status));
    }
    const dim3 grid(shape.heads, sequences, (shape.vdim + kColumns - 1) / kColumns);
    MB_LAUNCH("gated_delta_scan", (gated_delta_walk_kernel<T, kPer, kSplit>), dim3(grid), dim3(kColumns * kSplit), smem, stream, true, conv,
              conv_stride, (const T*)a_in, (const T*)b_in, in_stride, decay, dt_bias, state, state_stride, slots, cu_q, raw, shape);
    return check_launch("gated_delta_scan");
}

template <typename T>
int pick_delta_walk(const float* conv, int conv_stride, const void* a_in, const void* b_in, int in_stride, const float* decay,
                    const float* dt_bias, float* state, size_t state_stride, const int* slots, const int* cu_q,
                    int sequences, float* raw, DeltaShape shape, cudaStream_t stream) {
#define MB_DELTA(SPLIT, PER)                                                                                                          \
    if (shape.dim <= SPLIT * PER)                                                                                                     \
        return launch_delta_walk<T, PER, SPLIT>(conv, conv_stride, a_in, b_in, in_stride, decay, dt_bias, state, state_stride, \
                                                slots, cu_q, sequences, raw, shape, stream);
    MB_DELTA(4, 4)
    MB_DELTA(8, 4)
    MB_DELTA(8, 8)
    MB_DELTA(8, 16)
    MB_DELTA(8, 32)
#undef MB_DELTA
    return fail("gated_delta_scan: key heads of %d numbers exceed 256", shape.dim);
}

}  // namespace mb

using namespace mb;

// out [tokens, channels] float (row stride out_stride) = the convolution of the step's rows `in` (storage type, row stride
// in_stride) continued from every sequence's stored tail: state + slots[seq] * state_stride is [taps - 1][channels] floats.
// activation: 0 none, 1 silu.  store_tail != 0: the new tail is stored too (0: the state is left as it is).
// split (or null): bfloat16 [tokens][channels / per][2 * per], every result as its rounding and the rest.
MB_EXPORT int mb_short_conv(const void* in, int in_stride, int dtype, const float* in_bias, const float* weights, const float* out_bias,
                            int activation, float* out, int out_stride, float* state, size_t state_stride, const int* slots,
                            const int* cu_q, int sequences, int max_q_len, int channels, int taps, int store_tail, void* split, int per,
                            cudaStream_t stream) {
    if (sequences <= 0 || max_q_len <= 0 || channels <= 0) return 0;
    if (taps < 1 || taps > kMaxTaps) return fail("short_conv: %d taps are outside 1..%d", taps, kMaxTaps);
    if (sequences > 65535) return fail("short_conv: %d sequences exceed the grid limit 65535", sequences);
    if (split != nullptr && (per <= 0 || channels % per)) return fail("short_conv: %d channels are no whole blocks of %d", channels, per);
    const dim3 grid((channels + 127) / 128, (max_q_len + kConvTokens - 1) / kConvTokens, sequences);
    if (grid.y > 65535) return fail("short_conv: a step of %d tokens per sequence exceeds the grid", max_q_len);
    if (dtype == MB_F32)
        MB_LAUNCH("short_conv", short_conv_kernel<float>, dim3(grid), dim3(128), 0, stream, true, (const float*)in, in_stride, in_bias,
                  weights, out_bias, activation, out, out_stride, state, state_stride, slots, cu_q, channels, taps, store_tail,
                  (__nv_bfloat16*)split, per);
    else if (dtype == MB_BF16)
        MB_LAUNCH("short_conv", short_conv_kernel<__nv_bfloat16>, dim3(grid), dim3(128), 0, stream, true, (const __nv_bfloat16*)in,
                  in_stride, in_bias, weights, out_bias, activation, out, out_stride, state, state_stride, slots, cu_q, channels, taps,
                  store_tail, (__nv_bfloat16*)split, per);
    else
        return fail("short_conv: unknown dtype code %d", dtype);
    return check_launch("short_conv");
}

// conv: the convolved rows (float, row stride conv_stride; their q and k parts are made unit vectors in place) with q at column q_at (kv_heads heads of dim), k at k_at, v at v_at
// (heads heads of vdim); a_in, b_in [tokens, heads] and gate_in [tokens, heads * vdim] in the storage type with one row stride;
// decay (= -exp(A_log)), dt_bias [heads] and gain [vdim] float; state + slots[seq] * state_stride is [heads][dim][vdim] floats;
// raw: float scratch [tokens][heads * vdim] for the read-outs between the two kernels.
MB_EXPORT int mb_gated_delta_scan(float* conv, int conv_stride, const void* a_in, const void* b_in, const void* gate_in,
                                  int in_stride, int dtype, const float* decay, const float* dt_bias, const float* gain, float unit_eps,
                                  float eps, float* state, size_t state_stride, const int* slots, const int* cu_q, int sequences,
                                  int tokens, float* raw, void* out, int out_stride, float out_scale, int heads, int kv_heads, int dim,
                                  int vdim, int q_at, int k_at, int v_at, cudaStream_t stream) {
    if (sequences <= 0 || heads <= 0 || tokens <= 0) return 0;
    if (kv_heads <= 0 || heads % kv_heads) return fail("gated_delta_scan: %d heads are no multiple of %d query/key heads", heads, kv_heads);
    if (vdim <= 0 || vdim > 65535 * kColumns) return fail("gated_delta_scan: value heads of %d numbers", vdim);
    if (sequences > 65535) return fail("gated_delta_scan: %d sequences exceed the grid limit 65535", sequences);
    const DeltaShape shape{heads, kv_heads, dim, vdim, q_at, k_at, v_at};
    const int items = tokens * heads;
    const int unit_items = tokens * 2 * kv_heads;
    MB_LAUNCH("gated_delta_scan", unit_heads_kernel, dim3((unit_items + 3) / 4), dim3(128), 0, stream, true, conv, conv_stride, unit_items,
              unit_eps, shape);
    if (dtype == MB_F32) {
        if (int status = pick_delta_walk<float>(conv, conv_stride, a_in, b_in, in_stride, decay, dt_bias, state, state_stride, slots,
                                                cu_q, sequences, raw, shape, stream))
            return status;
        MB_LAUNCH("gated_delta_scan", head_norm_gate_kernel<float>, dim3((items + 3) / 4), dim3(128), 0, stream, true, raw,
                  (const float*)gate_in, in_stride, gain, eps, (float*)out, out_stride, out_scale, items, heads, vdim);
    } else if (dtype == MB_BF16) {
        if (int status = pick_delta_walk<__nv_bfloat16>(conv, conv_stride, a_in, b_in, in_stride, decay, dt_bias, state,
                                                        state_stride, slots, cu_q, sequences, raw, shape, stream))
            return status;
        MB_LAUNCH("gated_delta_scan", head_norm_gate_kernel<__nv_bfloat16>, dim3((items + 3) / 4), dim3(128), 0, stream, true, raw,
                  (const __nv_bfloat16*)gate_in, in_stride, gain, eps, (__nv_bfloat16*)out, out_stride, out_scale, items, heads, vdim);
    } else {
        return fail("gated_delta_scan: unknown dtype code %d", dtype);
    }
    return check_launch("gated_delta_scan");
}
