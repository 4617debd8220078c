// Short causal convolutions over time, and the gated delta rule; ragged sequences, per-sequence state kept in float.
//
// Short convolution, per channel c with `taps` weights w[c][0 .. taps - 1] whose LAST one meets the current token:
//   x_t = in_t (+ in_bias);   out_t = act(sum_i w[c][taps - 1 - i] x_(t - i) (+ out_bias)),   x = 0 before the sequence starts.
// The last taps - 1 inputs x of every sequence are part of its state: `tail` [taps - 1][channels], oldest first.  One kernel
// computes the new tokens' results from the stored tail and the step's inputs, a second one (launched after it) stores the
// new tail.
//
// Gated delta rule, per head h with its float state S [dim][vdim] (query/key head c = h / (heads / kv_heads)):
//   q_t, k_t: the convolved rows made unit vectors, x / sqrt(sum x^2 + unit_eps); q_t also times dim^(-1/2)
//   beta_t = sigmoid(b_t);   g_t = exp(decay_h * softplus(a_t + dt_bias_h))          (decay_h = -exp(A_log_h), a number <= 0)
//   S <- g_t S;   u = beta_t (v_t - S^T k_t);   S <- S + k_t u^T;   o_t = S^T q_t    (the read-out sees the token's own write)
//   out_t = out_scale * o_t / rms(o_t) * gain * silu(gate_t),   rms over the head's vdim numbers, gain [vdim] shared by the heads
// Everything after the projections is float arithmetic.  A block owns one (sequence, head); thread j keeps column j of S
// in registers and walks the tokens in groups of 8 whose rows pass through shared memory.
#include "common.cuh"

MB_DEFINE_LAST_ERROR()

namespace mb {

constexpr int kMaxTaps = 8;
constexpr int kConvTokens = 16;  // tokens a thread of the convolution walks
constexpr int kGroup = 8;        // tokens of a group of the delta rule's walk

__device__ __forceinline__ float sigmoid(float v) { return 1.0f / (1.0f + expf(-v)); }
__device__ __forceinline__ float softplus(float v) { return fmaxf(v, 0.0f) + log1pf(expf(-fabsf(v))); }

// grid (ceil(channels / 128), ceil(max_q_len / kConvTokens), sequences); block 128.
template <typename T>
__global__ void __launch_bounds__(128)
short_conv_kernel(const T* __restrict__ in, int in_stride, const float* __restrict__ in_bias, const float* __restrict__ weights,
                  const float* __restrict__ out_bias, int activation, float* __restrict__ out, int out_stride,
                  const float* __restrict__ state, size_t state_stride, const int* __restrict__ slots, const int* __restrict__ cu_q,
                  int channels, int taps) {
    grid_launch_dependents();
    grid_dependency_wait();
    const int c = blockIdx.x * blockDim.x + threadIdx.x, seq = blockIdx.z;
    const int first = cu_q[seq], count = cu_q[seq + 1] - first;
    const int j0 = blockIdx.y * kConvTokens, j1 = min(j0 + kConvTokens, count);
    if (c >= channels || j0 >= count) return;
    const float* tail = state + (size_t)slots[seq] * state_stride;
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
    for (int j = j0; j < j1; ++j) {
        x[0] = Num<T>::load(in + (size_t)(first + j) * in_stride + c) + bias_in;
        float sum = 0.0f;
#pragma unroll
        for (int i = kMaxTaps - 1; i >= 0; --i) sum = fmaf(w[i], x[i], sum);  // oldest input first
        sum += bias_out;
        if (activation == 1) sum = sum * sigmoid(sum);
        out[(size_t)(first + j) * out_stride + c] = sum;
#pragma unroll
        for (int i = kMaxTaps - 1; i >= 1; --i) x[i] = x[i - 1];
    }
}

// grid (ceil(channels / 128), sequences); block 128.  The new tail: the last taps - 1 inputs, taken from the step's tokens and,
// where the step brought fewer, from the old tail.
template <typename T>
__global__ void __launch_bounds__(128)
short_conv_tail_kernel(const T* __restrict__ in, int in_stride, const float* __restrict__ in_bias, float* __restrict__ state,
                       size_t state_stride, const int* __restrict__ slots, const int* __restrict__ cu_q, int channels, int taps) {
    grid_launch_dependents();
    grid_dependency_wait();
    const int c = blockIdx.x * blockDim.x + threadIdx.x, seq = blockIdx.y;
    const int first = cu_q[seq], count = cu_q[seq + 1] - first;
    if (c >= channels || count <= 0) return;
    float* tail = state + (size_t)slots[seq] * state_stride;
    const float bias_in = in_bias != nullptr ? in_bias[c] : 0.0f;
    float kept[kMaxTaps];
#pragma unroll
    for (int i = 0; i < kMaxTaps; ++i) {
        kept[i] = 0.0f;
        if (i < taps - 1) {
            const int j = count - (taps - 1) + i;
            kept[i] = j >= 0 ? Num<T>::load(in + (size_t)(first + j) * in_stride + c) + bias_in : tail[(size_t)(taps - 1 + j) * channels + c];
        }
    }
#pragma unroll
    for (int i = 0; i < kMaxTaps; ++i)
        if (i < taps - 1) tail[(size_t)i * channels + c] = kept[i];
}

struct DeltaShape {
    int heads, kv_heads, dim, vdim;
    int q_at, k_at, v_at;  // first columns of the convolved rows' q, k and v parts
};

// grid (heads, sequences); block: vdim rounded up to a multiple of 32.  kDim >= dim: the registers of a state column.
// shared: q [kGroup][kDim], k [kGroup][kDim], v [kGroup][vdim], o [kGroup][vdim], then 3 * kGroup floats.
template <typename T, int kDim>
__global__ void __launch_bounds__(256) gated_delta_scan_kernel(const float* __restrict__ conv, int conv_stride, const T* __restrict__ a_in,
                                        const T* __restrict__ b_in, const T* __restrict__ gate_in, int in_stride,
                                        const float* __restrict__ decay, const float* __restrict__ dt_bias,
                                        const float* __restrict__ gain, float unit_eps, float eps, float* __restrict__ state,
                                        size_t state_stride, const int* __restrict__ slots, const int* __restrict__ cu_q,
                                        T* __restrict__ out, int out_stride, float out_scale, DeltaShape shape) {
    grid_launch_dependents();
    grid_dependency_wait();
    extern __shared__ __align__(16) float delta_shared[];
    const int head = blockIdx.x, seq = blockIdx.y;
    const int first = cu_q[seq], count = cu_q[seq + 1] - first;
    if (count <= 0) return;
    const int dim = shape.dim, vdim = shape.vdim;
    const int qk_head = head / (shape.heads / shape.kv_heads);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, warps = blockDim.x >> 5;
    float* q_s = delta_shared;
    float* k_s = q_s + kGroup * kDim;
    float* v_s = k_s + kGroup * kDim;
    float* o_s = v_s + kGroup * vdim;
    float* beta_s = o_s + kGroup * vdim;
    float* g_s = beta_s + kGroup;
    const bool live = tid < vdim;
    float* stored = state + (size_t)slots[seq] * state_stride + (size_t)head * dim * vdim;
    float s[kDim];
#pragma unroll
    for (int d = 0; d < kDim; ++d) s[d] = (live && d < dim) ? stored[(size_t)d * vdim + tid] : 0.0f;
    const float head_decay = decay[head], head_dt = dt_bias[head];
    const float q_scale = 1.0f / sqrtf((float)dim);

    for (int t0 = 0; t0 < count; t0 += kGroup) {
        const int n = min(kGroup, count - t0);
        __syncthreads();  // the group before is finished with the shared rows
        for (int i = tid; i < n * kDim; i += blockDim.x) {
            const int u = i / kDim, d = i % kDim;
            const float* row = conv + (size_t)(first + t0 + u) * conv_stride;
            q_s[i] = d < dim ? row[shape.q_at + qk_head * dim + d] : 0.0f;
            k_s[i] = d < dim ? row[shape.k_at + qk_head * dim + d] : 0.0f;
        }
        if (live)
            for (int u = 0; u < n; ++u) v_s[u * vdim + tid] = conv[(size_t)(first + t0 + u) * conv_stride + shape.v_at + head * vdim + tid];
        if (tid < n) {
            const size_t at = (size_t)(first + t0 + tid) * in_stride + head;
            beta_s[tid] = sigmoid(Num<T>::load(b_in + at));
            g_s[tid] = expf(head_decay * softplus(Num<T>::load(a_in + at) + head_dt));
        }
        __syncthreads();
        for (int u = warp; u < n; u += warps) {  // unit vectors
            float qq = 0.0f, kk = 0.0f;
            for (int d = lane; d < dim; d += 32) {
                qq = fmaf(q_s[u * kDim + d], q_s[u * kDim + d], qq);
                kk = fmaf(k_s[u * kDim + d], k_s[u * kDim + d], kk);
            }
            const float q_factor = q_scale / sqrtf(warp_sum(qq) + unit_eps), k_factor = 1.0f / sqrtf(warp_sum(kk) + unit_eps);
            for (int d = lane; d < dim; d += 32) {
                q_s[u * kDim + d] *= q_factor;
                k_s[u * kDim + d] *= k_factor;
            }
        }
        __syncthreads();
        if (live) {
            for (int u = 0; u < n; ++u) {
                const float g = g_s[u];
                const float* k = k_s + u * kDim;
                const float* q = q_s + u * kDim;
                float seen = 0.0f;
#pragma unroll
                for (int d = 0; d < kDim; ++d) {
                    s[d] *= g;
                    seen = fmaf(s[d], k[d], seen);
                }
                const float write = beta_s[u] * (v_s[u * vdim + tid] - seen);
                float o = 0.0f;
#pragma unroll
                for (int d = 0; d < kDim; ++d) {
                    s[d] = fmaf(k[d], write, s[d]);
                    o = fmaf(s[d], q[d], o);
                }
                o_s[u * vdim + tid] = o;
            }
        }
        __syncthreads();
        for (int u = warp; u < n; u += warps) {  // every head's result over its root mean square, gain, gate
            float squares = 0.0f;
            for (int j = lane; j < vdim; j += 32) squares = fmaf(o_s[u * vdim + j], o_s[u * vdim + j], squares);
            const float inv = out_scale / sqrtf(warp_sum(squares) / (float)vdim + eps);
            const size_t token = first + t0 + u;
            for (int j = lane; j < vdim; j += 32) {
                const float z = Num<T>::load(gate_in + token * in_stride + (size_t)head * vdim + j);
                Num<T>::store(out + token * out_stride + (size_t)head * vdim + j, o_s[u * vdim + j] * inv * gain[j] * (z * sigmoid(z)));
            }
        }
    }
    if (live) {
#pragma unroll
        for (int d = 0; d < kDim; ++d)
            if (d < dim) stored[(size_t)d * vdim + tid] = s[d];
    }
}

template <typename T, int kDim>
int launch_delta_scan(const float* conv, int conv_stride, const void* a_in, const void* b_in, const void* gate_in, int in_stride,
                      const float* decay, const float* dt_bias, const float* gain, float unit_eps, float eps, float* state,
                      size_t state_stride, const int* slots, const int* cu_q, int sequences, void* out, int out_stride, float out_scale,
                      DeltaShape shape, cudaStream_t stream) {
    const int threads = (shape.vdim + 31) / 32 * 32;
    const size_t smem = sizeof(float) * ((size_t)kGroup * (2 * kDim + 2 * shape.vdim) + 3 * kGroup);
    if (smem > 48 * 1024) {
        cudaError_t status = cudaFuncSetAttribute(gated_delta_scan_kernel<T, kDim>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (status != cudaSuccess) return fail("gated_delta_scan: cannot reserve %zu bytes of shared memory: %s", smem, cudaGetErrorString(status));
    }
    MB_LAUNCH("gated_delta_scan", (gated_delta_scan_kernel<T, kDim>), dim3(shape.heads, sequences), dim3(threads), smem, stream, true, conv,
              conv_stride, (const T*)a_in, (const T*)b_in, (const T*)gate_in, in_stride, decay, dt_bias, gain, unit_eps, eps, state,
              state_stride, slots, cu_q, (T*)out, out_stride, out_scale, shape);
    return check_launch("gated_delta_scan");
}

template <typename T>
int pick_delta_scan(const float* conv, int conv_stride, const void* a_in, const void* b_in, const void* gate_in, int in_stride,
                    const float* decay, const float* dt_bias, const float* gain, float unit_eps, float eps, float* state,
                    size_t state_stride, const int* slots, const int* cu_q, int sequences, void* out, int out_stride, float out_scale,
                    DeltaShape shape, cudaStream_t stream) {
#define MB_DELTA(N)                                                                                                                   \
    if (shape.dim <= N)                                                                                                               \
        return launch_delta_scan<T, N>(conv, conv_stride, a_in, b_in, gate_in, in_stride, decay, dt_bias, gain, unit_eps, eps, state, \
                                       state_stride, slots, cu_q, sequences, out, out_stride, out_scale, shape, stream);
    MB_DELTA(16)
    MB_DELTA(32)
    MB_DELTA(64)
    MB_DELTA(128)
    MB_DELTA(256)
#undef MB_DELTA
    return fail("gated_delta_scan: key heads of %d numbers exceed 256", shape.dim);
}

}  // namespace mb

using namespace mb;

// out [tokens, channels] float (row stride out_stride) = the convolution of the step's rows `in` (storage type, row stride
// in_stride) continued from every sequence's stored tail: state + slots[seq] * state_stride is [taps - 1][channels] floats.
// activation: 0 none, 1 silu.  The tail is not changed: mb_short_conv_tail stores the new one afterwards.
MB_EXPORT int mb_short_conv(const void* in, int in_stride, int dtype, const float* in_bias, const float* weights, const float* out_bias,
                            int activation, float* out, int out_stride, const float* state, size_t state_stride, const int* slots,
                            const int* cu_q, int sequences, int max_q_len, int channels, int taps, cudaStream_t stream) {
    if (sequences <= 0 || max_q_len <= 0 || channels <= 0) return 0;
    if (taps < 1 || taps > kMaxTaps) return fail("short_conv: %d taps are outside 1..%d", taps, kMaxTaps);
    if (sequences > 65535) return fail("short_conv: %d sequences exceed the grid limit 65535", sequences);
    const dim3 grid((channels + 127) / 128, (max_q_len + kConvTokens - 1) / kConvTokens, sequences);
    if (grid.y > 65535) return fail("short_conv: a step of %d tokens per sequence exceeds the grid", max_q_len);
    if (dtype == MB_F32)
        MB_LAUNCH("short_conv", short_conv_kernel<float>, dim3(grid), dim3(128), 0, stream, true, (const float*)in, in_stride, in_bias,
                  weights, out_bias, activation, out, out_stride, state, state_stride, slots, cu_q, channels, taps);
    else if (dtype == MB_BF16)
        MB_LAUNCH("short_conv", short_conv_kernel<__nv_bfloat16>, dim3(grid), dim3(128), 0, stream, true, (const __nv_bfloat16*)in,
                  in_stride, in_bias, weights, out_bias, activation, out, out_stride, state, state_stride, slots, cu_q, channels, taps);
    else
        return fail("short_conv: unknown dtype code %d", dtype);
    return check_launch("short_conv");
}

MB_EXPORT int mb_short_conv_tail(const void* in, int in_stride, int dtype, const float* in_bias, float* state, size_t state_stride,
                                 const int* slots, const int* cu_q, int sequences, int channels, int taps, cudaStream_t stream) {
    if (sequences <= 0 || channels <= 0 || taps <= 1) return 0;
    if (taps > kMaxTaps) return fail("short_conv_tail: %d taps exceed %d", taps, kMaxTaps);
    if (sequences > 65535) return fail("short_conv_tail: %d sequences exceed the grid limit 65535", sequences);
    const dim3 grid((channels + 127) / 128, sequences);
    if (dtype == MB_F32)
        MB_LAUNCH("short_conv_tail", short_conv_tail_kernel<float>, dim3(grid), dim3(128), 0, stream, true, (const float*)in, in_stride,
                  in_bias, state, state_stride, slots, cu_q, channels, taps);
    else if (dtype == MB_BF16)
        MB_LAUNCH("short_conv_tail", short_conv_tail_kernel<__nv_bfloat16>, dim3(grid), dim3(128), 0, stream, true,
                  (const __nv_bfloat16*)in, in_stride, in_bias, state, state_stride, slots, cu_q, channels, taps);
    else
        return fail("short_conv_tail: unknown dtype code %d", dtype);
    return check_launch("short_conv_tail");
}

// conv: the convolved rows (float, row stride conv_stride) with q at column q_at (kv_heads heads of dim), k at k_at, v at v_at
// (heads heads of vdim); a_in, b_in [tokens, heads] and gate_in [tokens, heads * vdim] in the storage type with one row stride;
// decay (= -exp(A_log)), dt_bias [heads] and gain [vdim] float; state + slots[seq] * state_stride is [heads][dim][vdim] floats.
MB_EXPORT int mb_gated_delta_scan(const float* conv, int conv_stride, const void* a_in, const void* b_in, const void* gate_in,
                                  int in_stride, int dtype, const float* decay, const float* dt_bias, const float* gain, float unit_eps,
                                  float eps, float* state, size_t state_stride, const int* slots, const int* cu_q, int sequences,
                                  void* out, int out_stride, float out_scale, int heads, int kv_heads, int dim, int vdim, int q_at,
                                  int k_at, int v_at, cudaStream_t stream) {
    if (sequences <= 0 || heads <= 0) return 0;
    if (kv_heads <= 0 || heads % kv_heads) return fail("gated_delta_scan: %d heads are no multiple of %d query/key heads", heads, kv_heads);
    if (vdim <= 0 || vdim > 256) return fail("gated_delta_scan: value heads of %d numbers are outside 1..256", vdim);
    if (sequences > 65535) return fail("gated_delta_scan: %d sequences exceed the grid limit 65535", sequences);
    const DeltaShape shape{heads, kv_heads, dim, vdim, q_at, k_at, v_at};
    if (dtype == MB_F32)
        return pick_delta_scan<float>(conv, conv_stride, a_in, b_in, gate_in, in_stride, decay, dt_bias, gain, unit_eps, eps, state,
                                      state_stride, slots, cu_q, sequences, out, out_stride, out_scale, shape, stream);
    if (dtype == MB_BF16)
        return pick_delta_scan<__nv_bfloat16>(conv, conv_stride, a_in, b_in, gate_in, in_stride, decay, dt_bias, gain, unit_eps, eps, state,
                                              state_stride, slots, cu_q, sequences, out, out_stride, out_scale, shape, stream);
    return fail("gated_delta_scan: unknown dtype code %d", dtype);
}
