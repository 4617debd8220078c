// Element-wise gated recurrences over the tokens of ragged sequences, with the state of every sequence
// kept in float between steps.
//
// minGRU (gates read the current token only):
//   z_t = sigmoid(zin_t + bz)          u_t = xin_t + bx
//   c_t = u_t + 1/2 where u_t >= 0, sigmoid(u_t) elsewhere
//   S_t = (1 - z_t) S_(t-1) + z_t c_t
//   y_t = out_scale * S_t * silu(gin_t)
// zin, xin, gin are projections of the token (storage type, float or bfloat16); everything after them is float.
//
// The recurrence is linear in S, so a step of many tokens is cut into `chunks` runs of consecutive tokens
// that are walked at the same time: each run first finds its own (A, B) with S_end = A S_start + B, the
// starts follow from the sequence's stored state by composing the runs before, and a second walk writes
// the results.  With one token per sequence (decoding) there is one run and one walk.
//
// Real-gated linear recurrent unit (gates read the convolved input u of the current token, through one small square matrix
// per block of channels whose sums arrive as r_in and i_in):
//   r_t = sigmoid(r_in_t + br)         i_t = sigmoid(i_in_t + bi)
//   log a_t = rate * r_t   (rate = -c softplus(lambda) per channel, a number <= 0)        a_t = exp(log a_t)
//   S_t = a_t S_(t-1) + sqrt(1 - a_t^2) i_t u_t                  (1 - a^2 is taken as -expm1(2 log a))
//   y_t = out_scale * S_t * gelu_tanh(y_in_t + by)
// r_in, i_in and u are float rows; y_in is a projection in the storage type.  The same runs and two walks as above.
#include "common.cuh"

MB_DEFINE_LAST_ERROR()

namespace mb {

constexpr int kBlockThreads = 1024;  // channels of a block times runs of a block, at most
constexpr int kMaxChunks = 128;
constexpr int kKeep = 16;  // tokens of a run whose gates and candidates stay in registers between the walks

__device__ __forceinline__ float sigmoid(float v) { return 1.0f / (1.0f + expf(-v)); }

// grid (ceil(width / channels), sequences); block (channels, chunks) with channels * chunks <= 1024.
template <typename T>
__global__ void __launch_bounds__(kBlockThreads) mingru_scan_kernel(const T* __restrict__ zin, const T* __restrict__ xin, const T* __restrict__ gin,
                                   int in_stride, const float* __restrict__ z_bias, const float* __restrict__ x_bias,
                                   float* __restrict__ state, const int* __restrict__ slots, const int* __restrict__ cu_q,
                                   int width, T* __restrict__ out, int out_stride, float out_scale) {
    grid_launch_dependents();
    grid_dependency_wait();
    __shared__ float a_of[kBlockThreads];  // [run][channel of the block]
    __shared__ float b_of[kBlockThreads];
    const int seq = blockIdx.y;
    const int first = cu_q[seq];
    const int count = cu_q[seq + 1] - first;
    if (count <= 0) return;  // the whole block leaves
    const int channel = blockIdx.x * blockDim.x + threadIdx.x;
    const bool live = channel < width;
    const int chunks = blockDim.y, chunk = threadIdx.y;
    const int per = (count + chunks - 1) / chunks;
    const int t0 = min(chunk * per, count), t1 = min(t0 + per, count);
    const float bz = live ? z_bias[channel] : 0.0f, bx = live ? x_bias[channel] : 0.0f;

    if (chunks > 1 && per <= kKeep) {
        // Short runs (the usual case: the launcher cuts a prompt into runs of about 16 tokens): every input of the
        // run is asked for at once, and the gates and candidates of the first walk stay in registers for the
        // second, which then reads only the output gates.  A token beyond the run has z = 0: it changes nothing.
        float zk[kKeep], ck[kKeep];
        if (live) {
#pragma unroll
            for (int half = 0; half < kKeep; half += kKeep / 2) {  // (eight tokens' loads at a time: registers)
                float zr[kKeep / 2], xr[kKeep / 2];
#pragma unroll
                for (int u = 0; u < kKeep / 2; ++u) {
                    const size_t at = (size_t)(first + min(t0 + half + u, count - 1)) * in_stride + channel;
                    zr[u] = Num<T>::load(zin + at);
                    xr[u] = Num<T>::load(xin + at);
                }
#pragma unroll
                for (int u = 0; u < kKeep / 2; ++u) {
                    const float x = xr[u] + bx;
                    zk[half + u] = t0 + half + u < t1 ? sigmoid(zr[u] + bz) : 0.0f;
                    ck[half + u] = x >= 0.0f ? x + 0.5f : sigmoid(x);
                }
            }
        }
        float a = 1.0f, b = 0.0f;
        if (live) {
#pragma unroll
            for (int u = 0; u < kKeep; ++u) {
                a *= 1.0f - zk[u];
                b = (1.0f - zk[u]) * b + zk[u] * ck[u];
            }
        }
        a_of[chunk * blockDim.x + threadIdx.x] = a;
        b_of[chunk * blockDim.x + threadIdx.x] = b;
        __syncthreads();
        if (!live) return;
        float* stored = state + (size_t)slots[seq] * width + channel;
        float s = *stored;
        for (int before = 0; before < chunk; ++before) s = a_of[before * blockDim.x + threadIdx.x] * s + b_of[before * blockDim.x + threadIdx.x];
#pragma unroll
        for (int half = 0; half < kKeep; half += kKeep / 2) {
            float gr[kKeep / 2];
#pragma unroll
            for (int u = 0; u < kKeep / 2; ++u)
                gr[u] = Num<T>::load(gin + (size_t)(first + min(t0 + half + u, count - 1)) * in_stride + channel);
#pragma unroll
            for (int u = 0; u < kKeep / 2; ++u) {
                s = (1.0f - zk[half + u]) * s + zk[half + u] * ck[half + u];
                if (t0 + half + u < t1)
                    Num<T>::store(out + (size_t)(first + t0 + half + u) * out_stride + channel, out_scale * s * (gr[u] * sigmoid(gr[u])));
            }
        }
        if (chunk == chunks - 1) *stored = s;
        return;
    }
    // Longer runs: loads do not depend on the recurrence, so eight tokens' inputs are asked for before the first is used.
    constexpr int kAhead = 8;
    if (chunks > 1) {
        float a = 1.0f, b = 0.0f;
        if (live) {
            int t = t0;
            for (; t + kAhead <= t1; t += kAhead) {
                float zr[kAhead], xr[kAhead];
#pragma unroll
                for (int u = 0; u < kAhead; ++u) {
                    const size_t at = (size_t)(first + t + u) * in_stride + channel;
                    zr[u] = Num<T>::load(zin + at);
                    xr[u] = Num<T>::load(xin + at);
                }
#pragma unroll
                for (int u = 0; u < kAhead; ++u) {
                    const float z = sigmoid(zr[u] + bz), x = xr[u] + bx;
                    const float c = x >= 0.0f ? x + 0.5f : sigmoid(x);
                    a *= 1.0f - z;
                    b = (1.0f - z) * b + z * c;
                }
            }
            for (; t < t1; ++t) {
                const size_t at = (size_t)(first + t) * in_stride + channel;
                const float z = sigmoid(Num<T>::load(zin + at) + bz);
                const float x = Num<T>::load(xin + at) + bx;
                const float c = x >= 0.0f ? x + 0.5f : sigmoid(x);
                a *= 1.0f - z;
                b = (1.0f - z) * b + z * c;
            }
        }
        a_of[chunk * blockDim.x + threadIdx.x] = a;
        b_of[chunk * blockDim.x + threadIdx.x] = b;
        __syncthreads();
    }
    if (!live) return;
    float* stored = state + (size_t)slots[seq] * width + channel;
    float s = *stored;
    for (int before = 0; before < chunk; ++before) s = a_of[before * blockDim.x + threadIdx.x] * s + b_of[before * blockDim.x + threadIdx.x];
    int t = t0;
    for (; t + kAhead <= t1; t += kAhead) {
        float zr[kAhead], xr[kAhead], gr[kAhead];
#pragma unroll
        for (int u = 0; u < kAhead; ++u) {
            const size_t at = (size_t)(first + t + u) * in_stride + channel;
            zr[u] = Num<T>::load(zin + at);
            xr[u] = Num<T>::load(xin + at);
            gr[u] = Num<T>::load(gin + at);
        }
#pragma unroll
        for (int u = 0; u < kAhead; ++u) {
            const float z = sigmoid(zr[u] + bz), x = xr[u] + bx;
            const float c = x >= 0.0f ? x + 0.5f : sigmoid(x);
            s = (1.0f - z) * s + z * c;
            Num<T>::store(out + (size_t)(first + t + u) * out_stride + channel, out_scale * s * (gr[u] * sigmoid(gr[u])));
        }
    }
    for (; t < t1; ++t) {
        const size_t at = (size_t)(first + t) * in_stride + channel;
        const float z = sigmoid(Num<T>::load(zin + at) + bz);
        const float x = Num<T>::load(xin + at) + bx;
        const float c = x >= 0.0f ? x + 0.5f : sigmoid(x);
        s = (1.0f - z) * s + z * c;
        const float g = Num<T>::load(gin + at);
        Num<T>::store(out + (size_t)(first + t) * out_stride + channel, out_scale * s * (g * sigmoid(g)));
    }
    if (chunk == chunks - 1) *stored = s;  // runs after the last token are empty: this is the state after all of them
}

struct RglruCell {
    float a, b;
};

// the gate sums of channel c lie block by block: [r of block 0 | i of block 0 | r of block 1 | ...], `per` channels a block
__device__ __forceinline__ RglruCell rglru_cell(float r_sum, float i_sum, float u, float br, float bi, float rate) {
    const float r = sigmoid(r_sum + br), i = sigmoid(i_sum + bi);
    const float log_a = rate * r;
    return RglruCell{expf(log_a), sqrtf(-expm1f(2.0f * log_a)) * i * u};
}

// grid (ceil(width / channels), sequences); block (channels, chunks) with channels * chunks <= 1024.
template <typename T>
__global__ void __launch_bounds__(kBlockThreads) rglru_scan_kernel(const float* __restrict__ gates, int gate_stride, int per,
                                  const float* __restrict__ u, int u_stride, const T* __restrict__ y_in, int y_stride,
                                  const float* __restrict__ r_bias, const float* __restrict__ i_bias, const float* __restrict__ y_bias,
                                  const float* __restrict__ rate, float* __restrict__ state, size_t state_stride,
                                  const int* __restrict__ slots, const int* __restrict__ cu_q, int width, T* __restrict__ out,
                                  int out_stride, float out_scale) {
    grid_launch_dependents();
    grid_dependency_wait();
    __shared__ float a_of[kBlockThreads];  // [run][channel of the block]
    __shared__ float b_of[kBlockThreads];
    const int seq = blockIdx.y;
    const int first = cu_q[seq];
    const int count = cu_q[seq + 1] - first;
    if (count <= 0) return;  // the whole block leaves
    const int channel = blockIdx.x * blockDim.x + threadIdx.x;
    const bool live = channel < width;
    const int chunks = blockDim.y, chunk = threadIdx.y;
    const int per_run = (count + chunks - 1) / chunks;
    const int t0 = min(chunk * per_run, count), t1 = min(t0 + per_run, count);
    const int c = live ? channel : 0;
    const float br = r_bias[c], bi = i_bias[c], by = y_bias[c], channel_rate = rate[c];
    const int r_at = (c / per) * 2 * per + c % per, i_at = r_at + per;
    constexpr int kAhead = 8;  // loads do not depend on the recurrence: eight tokens' inputs are asked for before the first is used
    if (chunks > 1) {
        float a = 1.0f, b = 0.0f;
        if (live) {
            for (int t = t0; t < t1; t += kAhead) {
                float rr[kAhead], ir[kAhead], ur[kAhead];
#pragma unroll
                for (int k = 0; k < kAhead; ++k) {
                    const size_t token = first + min(t + k, t1 - 1);
                    rr[k] = gates[token * gate_stride + r_at];
                    ir[k] = gates[token * gate_stride + i_at];
                    ur[k] = u[token * u_stride + c];
                }
#pragma unroll
                for (int k = 0; k < kAhead; ++k) {
                    if (t + k >= t1) break;
                    const RglruCell cell = rglru_cell(rr[k], ir[k], ur[k], br, bi, channel_rate);
                    a *= cell.a;
                    b = cell.a * b + cell.b;
                }
            }
        }
        a_of[chunk * blockDim.x + threadIdx.x] = a;
        b_of[chunk * blockDim.x + threadIdx.x] = b;
        __syncthreads();
    }
    if (!live) return;
    float* stored = state + (size_t)slots[seq] * state_stride + channel;
    float s = *stored;
    for (int before = 0; before < chunk; ++before) s = a_of[before * blockDim.x + threadIdx.x] * s + b_of[before * blockDim.x + threadIdx.x];
    for (int t = t0; t < t1; t += kAhead) {
        float rr[kAhead], ir[kAhead], ur[kAhead], yr[kAhead];
#pragma unroll
        for (int k = 0; k < kAhead; ++k) {
            const size_t token = first + min(t + k, t1 - 1);
            rr[k] = gates[token * gate_stride + r_at];
            ir[k] = gates[token * gate_stride + i_at];
            ur[k] = u[token * u_stride + c];
            yr[k] = Num<T>::load(y_in + token * y_stride + c);
        }
#pragma unroll
        for (int k = 0; k < kAhead; ++k) {
            if (t + k >= t1) break;
            const RglruCell cell = rglru_cell(rr[k], ir[k], ur[k], br, bi, channel_rate);
            s = cell.a * s + cell.b;
            Num<T>::store(out + (size_t)(first + t + k) * out_stride + c, out_scale * s * gate_activation(MB_ACT_GELU_TANH, yr[k] + by));
        }
    }
    if (chunk == chunks - 1) *stored = s;  // runs after the last token are empty: this is the state after all of them
}

}  // namespace mb

using namespace mb;

// zin, xin, gin: [tokens, >= width] rows of the storage type with one row stride (column slices of one
// tensor); out likewise with its own stride.  state: float [slots, width]; slots[sequence] picks the row.
MB_EXPORT int mb_mingru_scan(const void* zin, const void* xin, const void* gin, int in_stride, int dtype,
                             const float* z_bias, const float* x_bias, float* state, const int* slots, const int* cu_q,
                             int sequences, int max_q_len, int width, void* out, int out_stride, float out_scale,
                             cudaStream_t stream) {
    if (sequences <= 0 || max_q_len <= 0 || width <= 0) return 0;
    if (sequences > 65535) return fail("mingru_scan: %d sequences exceed the grid limit 65535", sequences);
    // Runs of about 16 tokens, so that a long prompt is walked by many threads at once; the fewer channels a block
    // then has (down to 8, which still fills a 16-byte piece of a bfloat16 row), the more blocks there are.
    int chunks = 1;
    while (chunks < kMaxChunks && chunks * 16 < max_q_len) chunks *= 2;
    int channels = chunks == 1 ? 128 : kBlockThreads / chunks;
    if (channels > 32 && chunks > 1) channels = 32;
    const dim3 grid((width + channels - 1) / channels, sequences), block(channels, chunks);
    if (dtype == MB_F32)
        MB_LAUNCH("mingru_scan", mingru_scan_kernel<float>, dim3(grid), dim3(block), 0, stream, true,
                  (const float*)zin, (const float*)xin, (const float*)gin, in_stride, z_bias, x_bias, state, slots,
                  cu_q, width, (float*)out, out_stride, out_scale);
    else if (dtype == MB_BF16)
        MB_LAUNCH("mingru_scan", mingru_scan_kernel<__nv_bfloat16>, dim3(grid), dim3(block), 0, stream, true,
                  (const __nv_bfloat16*)zin, (const __nv_bfloat16*)xin, (const __nv_bfloat16*)gin, in_stride, z_bias,
                  x_bias, state, slots, cu_q, width, (__nv_bfloat16*)out, out_stride, out_scale);
    else
        return fail("mingru_scan: unknown dtype code %d", dtype);
    return check_launch("mingru_scan");
}

// gates: float [tokens, 2 * width] block by block (r sums then i sums of each block of `per` channels); u float [tokens, width];
// y_in [tokens, width] in the storage type; biases and rate float [width]; state + slots[seq] * state_stride is [width] floats.
MB_EXPORT int mb_rglru_scan(const float* gates, int gate_stride, int per, const float* u, int u_stride, const void* y_in, int y_stride,
                            int dtype, const float* r_bias, const float* i_bias, const float* y_bias, const float* rate, float* state,
                            size_t state_stride, const int* slots, const int* cu_q, int sequences, int max_q_len, int width, void* out,
                            int out_stride, float out_scale, cudaStream_t stream) {
    if (sequences <= 0 || max_q_len <= 0 || width <= 0) return 0;
    if (sequences > 65535) return fail("rglru_scan: %d sequences exceed the grid limit 65535", sequences);
    if (per <= 0 || width % per) return fail("rglru_scan: %d channels are no whole blocks of %d", width, per);
    int chunks = 1;
    while (chunks < kMaxChunks && chunks * 16 < max_q_len) chunks *= 2;
    int channels = chunks == 1 ? 128 : kBlockThreads / chunks;
    if (channels > 32 && chunks > 1) channels = 32;
    const dim3 grid((width + channels - 1) / channels, sequences), block(channels, chunks);
    if (dtype == MB_F32)
        MB_LAUNCH("rglru_scan", rglru_scan_kernel<float>, dim3(grid), dim3(block), 0, stream, true, gates, gate_stride, per, u, u_stride,
                  (const float*)y_in, y_stride, r_bias, i_bias, y_bias, rate, state, state_stride, slots, cu_q, width, (float*)out,
                  out_stride, out_scale);
    else if (dtype == MB_BF16)
        MB_LAUNCH("rglru_scan", rglru_scan_kernel<__nv_bfloat16>, dim3(grid), dim3(block), 0, stream, true, gates, gate_stride, per, u,
                  u_stride, (const __nv_bfloat16*)y_in, y_stride, r_bias, i_bias, y_bias, rate, state, state_stride, slots, cu_q, width,
                  (__nv_bfloat16*)out, out_stride, out_scale);
    else
        return fail("rglru_scan: unknown dtype code %d", dtype);
    return check_launch("rglru_scan");
}
