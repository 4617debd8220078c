// Several copies of the residual stream side by side (hyper-connections): x [tokens][streams][width], float.
//
//   read:   u = sum_s in[s] x_s;  out = u / sqrt(mean(u^2) + eps) * gain           (the norm a sublayer reads through)
//   write:  x_t <- sum_s mix[s][t] x_s + out[t] * y   for all t at once, from the old copies
//   copies: every copy starts as the embedding's row;  sum: the copies added up (what the final norm reads)
//
// All arithmetic is float; `out` of read and `y` of write are float or bfloat16.
#include "common.cuh"

MB_DEFINE_LAST_ERROR()

namespace mb {

constexpr int kMaxStreams = 8;

// grid (ceil(tokens * width / 256)); block 256.
__global__ void stream_copies_kernel(const float* __restrict__ x, float* __restrict__ out, size_t total, int width, int streams) {
    grid_launch_dependents();
    grid_dependency_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const size_t t = i / width;
    const int c = (int)(i % width);
    const float v = x[i];
    for (int s = 0; s < streams; ++s) out[(t * streams + s) * width + c] = v;
}

__global__ void stream_sum_kernel(const float* __restrict__ x, float* __restrict__ out, size_t total, int width, int streams) {
    grid_launch_dependents();
    grid_dependency_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const size_t t = i / width;
    const int c = (int)(i % width);
    float sum = 0.0f;
    for (int s = 0; s < streams; ++s) sum += x[(t * streams + s) * width + c];
    out[i] = sum;
}

__device__ __forceinline__ void store4(float* p, float a, float b, float c, float d) { *reinterpret_cast<float4*>(p) = make_float4(a, b, c, d); }
__device__ __forceinline__ void store4(__nv_bfloat16* p, float a, float b, float c, float d) {
    const __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
    *reinterpret_cast<uint2*>(p) = make_uint2(*reinterpret_cast<const uint32_t*>(&lo), *reinterpret_cast<const uint32_t*>(&hi));
}

// grid (rows); block 256; shared: width floats + 32.  `in` holds the streams' read coefficients on the device.
// kQuads: width is a multiple of 4; a thread reads four columns of every stream with one 16-byte load each, all streams'
// loads of a step in flight together.
template <typename T, bool kQuads>
__global__ void __launch_bounds__(256)
hyper_read_norm_kernel(const float* __restrict__ x, const float* __restrict__ in, const float* __restrict__ gain,
                       T* __restrict__ out, int width, int streams, float eps) {
    grid_launch_dependents();
    extern __shared__ __align__(16) float row_shared[];
    float* scratch = row_shared + width;
    float coefficient[kMaxStreams];
#pragma unroll
    for (int s = 0; s < kMaxStreams; ++s) coefficient[s] = s < streams ? in[s] : 0.0f;  // (weights: written before the step)
    grid_dependency_wait();
    const size_t row = blockIdx.x;
    const float* mine = x + row * streams * width;
    float ssq = 0.0f;
    if (kQuads) {
        const int quads = width / 4;
        for (int c = threadIdx.x; c < quads; c += blockDim.x) {
            float4 v[kMaxStreams];
#pragma unroll
            for (int s = 0; s < kMaxStreams; ++s)
                if (s < streams) v[s] = reinterpret_cast<const float4*>(mine + (size_t)s * width)[c];
            float4 u = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
            for (int s = 0; s < kMaxStreams; ++s)
                if (s < streams) {
                    u.x = fmaf(coefficient[s], v[s].x, u.x);
                    u.y = fmaf(coefficient[s], v[s].y, u.y);
                    u.z = fmaf(coefficient[s], v[s].z, u.z);
                    u.w = fmaf(coefficient[s], v[s].w, u.w);
                }
            reinterpret_cast<float4*>(row_shared)[c] = u;
            ssq = fmaf(u.x, u.x, fmaf(u.y, u.y, fmaf(u.z, u.z, fmaf(u.w, u.w, ssq))));
        }
    } else {
        for (int c = threadIdx.x; c < width; c += blockDim.x) {
            float u = 0.0f;
#pragma unroll
            for (int s = 0; s < kMaxStreams; ++s)
                if (s < streams) u = fmaf(coefficient[s], mine[(size_t)s * width + c], u);
            row_shared[c] = u;
            ssq = fmaf(u, u, ssq);
        }
    }
    const float total = block_sum(ssq, scratch);
    const float inverse = 1.0f / sqrtf(total / (float)width + eps);
    if (kQuads) {
        for (int c = threadIdx.x; c < width / 4; c += blockDim.x) {
            const float4 u = reinterpret_cast<const float4*>(row_shared)[c];
            const float4 g = reinterpret_cast<const float4*>(gain)[c];
            store4(out + row * width + c * 4, u.x * inverse * g.x, u.y * inverse * g.y, u.z * inverse * g.z, u.w * inverse * g.w);
        }
    } else {
        for (int c = threadIdx.x; c < width; c += blockDim.x) Num<T>::store(out + row * width + c, row_shared[c] * inverse * gain[c]);
    }
}

// grid (ceil(tokens * width / 256)); block 256.  `coefficients`: out [streams] then mix [streams][streams] on the device.
template <typename T>
__global__ void __launch_bounds__(256)
hyper_write_kernel(float* __restrict__ x, const T* __restrict__ y, int y_stride, const float* __restrict__ out_coefficients,
                   const float* __restrict__ mix, size_t total, int width, int streams) {
    grid_launch_dependents();
    __shared__ float mix_shared[kMaxStreams * kMaxStreams + kMaxStreams];
    if (threadIdx.x < streams * streams) mix_shared[threadIdx.x] = mix[threadIdx.x];
    if (threadIdx.x < streams) mix_shared[kMaxStreams * kMaxStreams + threadIdx.x] = out_coefficients[threadIdx.x];
    __syncthreads();
    grid_dependency_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const size_t t = i / width;
    const int c = (int)(i % width);
    float* mine = x + t * streams * width + c;
    float old[kMaxStreams];
#pragma unroll
    for (int s = 0; s < kMaxStreams; ++s) old[s] = s < streams ? mine[(size_t)s * width] : 0.0f;
    const float added = Num<T>::load(y + t * y_stride + c);
#pragma unroll
    for (int to = 0; to < kMaxStreams; ++to) {
        if (to < streams) {
            float value = mix_shared[kMaxStreams * kMaxStreams + to] * added;
#pragma unroll
            for (int from = 0; from < kMaxStreams; ++from)
                if (from < streams) value = fmaf(mix_shared[from * streams + to], old[from], value);
            mine[(size_t)to * width] = value;
        }
    }
}

// Writing one sublayer's result and reading for the next in one pass over the row: the new copies are stored and the next
// sublayer's weighted sum is taken from them while they are in registers, so the copies are read once, not twice.  Every
// number is computed in the order of hyper_write_kernel followed by hyper_read_norm_kernel: the same bits as the two kernels.
// grid (rows); block 256; shared: width floats + 32.
template <typename T, bool kQuads>
__global__ void __launch_bounds__(256)
hyper_write_read_norm_kernel(float* __restrict__ x, const float* __restrict__ y, int y_stride, const float* __restrict__ out_coefficients,
                             const float* __restrict__ mix, const float* __restrict__ in, const float* __restrict__ gain,
                             T* __restrict__ out, int width, int streams, float eps) {
    grid_launch_dependents();
    extern __shared__ __align__(16) float row_shared[];
    float* scratch = row_shared + width;
    __shared__ float mix_shared[kMaxStreams * kMaxStreams + 2 * kMaxStreams];
    if (threadIdx.x < streams * streams) mix_shared[threadIdx.x] = mix[threadIdx.x];
    if (threadIdx.x < streams) {
        mix_shared[kMaxStreams * kMaxStreams + threadIdx.x] = out_coefficients[threadIdx.x];
        mix_shared[kMaxStreams * kMaxStreams + kMaxStreams + threadIdx.x] = in[threadIdx.x];
    }
    __syncthreads();  // (weights: written before the step)
    grid_dependency_wait();
    const float* out_c = mix_shared + kMaxStreams * kMaxStreams;
    const float* in_c = out_c + kMaxStreams;
    const size_t row = blockIdx.x;
    float* mine = x + row * streams * width;
    const float* added_row = y + row * y_stride;
    float ssq = 0.0f;
    if (kQuads) {
        for (int c = threadIdx.x; c < width / 4; c += blockDim.x) {
            float4 v[kMaxStreams];
#pragma unroll
            for (int s = 0; s < kMaxStreams; ++s)
                if (s < streams) v[s] = reinterpret_cast<const float4*>(mine + (size_t)s * width)[c];
            const float4 added = reinterpret_cast<const float4*>(added_row)[c];
            float4 u = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
            for (int to = 0; to < kMaxStreams; ++to) {
                if (to < streams) {
                    float4 value = make_float4(out_c[to] * added.x, out_c[to] * added.y, out_c[to] * added.z, out_c[to] * added.w);
#pragma unroll
                    for (int from = 0; from < kMaxStreams; ++from)
                        if (from < streams) {
                            const float m = mix_shared[from * streams + to];
                            value.x = fmaf(m, v[from].x, value.x);
                            value.y = fmaf(m, v[from].y, value.y);
                            value.z = fmaf(m, v[from].z, value.z);
                            value.w = fmaf(m, v[from].w, value.w);
                        }
                    reinterpret_cast<float4*>(mine + (size_t)to * width)[c] = value;
                    u.x = fmaf(in_c[to], value.x, u.x);
                    u.y = fmaf(in_c[to], value.y, u.y);
                    u.z = fmaf(in_c[to], value.z, u.z);
                    u.w = fmaf(in_c[to], value.w, u.w);
                }
            }
            reinterpret_cast<float4*>(row_shared)[c] = u;
            ssq = fmaf(u.x, u.x, fmaf(u.y, u.y, fmaf(u.z, u.z, fmaf(u.w, u.w, ssq))));
        }
    } else {
        for (int c = threadIdx.x; c < width; c += blockDim.x) {
            float old[kMaxStreams];
#pragma unroll
            for (int s = 0; s < kMaxStreams; ++s) old[s] = s < streams ? mine[(size_t)s * width + c] : 0.0f;
            const float added = added_row[c];
            float u = 0.0f;
#pragma unroll
            for (int to = 0; to < kMaxStreams; ++to) {
                if (to < streams) {
                    float value = out_c[to] * added;
#pragma unroll
                    for (int from = 0; from < kMaxStreams; ++from)
                        if (from < streams) value = fmaf(mix_shared[from * streams + to], old[from], value);
                    mine[(size_t)to * width + c] = value;
                    u = fmaf(in_c[to], value, u);
                }
            }
            row_shared[c] = u;
            ssq = fmaf(u, u, ssq);
        }
    }
    const float total = block_sum(ssq, scratch);
    const float inverse = 1.0f / sqrtf(total / (float)width + eps);
    if (kQuads) {
        for (int c = threadIdx.x; c < width / 4; c += blockDim.x) {
            const float4 u = reinterpret_cast<const float4*>(row_shared)[c];
            const float4 g = reinterpret_cast<const float4*>(gain)[c];
            store4(out + row * width + c * 4, u.x * inverse * g.x, u.y * inverse * g.y, u.z * inverse * g.z, u.w * inverse * g.w);
        }
    } else {
        for (int c = threadIdx.x; c < width; c += blockDim.x) Num<T>::store(out + row * width + c, row_shared[c] * inverse * gain[c]);
    }
}

}  // namespace mb

using namespace mb;

MB_EXPORT int mb_hyper_max_streams() { return kMaxStreams; }

// out [tokens][streams][width] <- x [tokens][width], every copy.
MB_EXPORT int mb_stream_copies(const float* x, float* out, int tokens, int width, int streams, cudaStream_t stream) {
    if (tokens <= 0) return 0;
    if (width <= 0 || streams <= 0) return fail("stream_copies: width %d, streams %d", width, streams);
    const size_t total = (size_t)tokens * width;
    MB_LAUNCH("stream_copies", stream_copies_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, stream, true, x, out, total, width, streams);
    return 0;
}

MB_EXPORT int mb_stream_sum(const float* x, float* out, int tokens, int width, int streams, cudaStream_t stream) {
    if (tokens <= 0) return 0;
    if (width <= 0 || streams <= 0) return fail("stream_sum: width %d, streams %d", width, streams);
    const size_t total = (size_t)tokens * width;
    MB_LAUNCH("stream_sum", stream_sum_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, stream, true, x, out, total, width, streams);
    return 0;
}

MB_EXPORT int mb_hyper_read_norm(const float* x, const float* in, const float* gain, void* out, int out_dtype, int tokens, int width,
                                 int streams, float eps, cudaStream_t stream) {
    if (tokens <= 0) return 0;
    if (width <= 0 || streams <= 0 || streams > kMaxStreams) return fail("hyper_read_norm: width %d, streams %d (at most %d)", width, streams, kMaxStreams);
    const size_t smem = ((size_t)width + 32) * sizeof(float);
    if (smem > 200 * 1024) return fail("hyper_read_norm: a row of %d floats exceeds a block's shared memory", width);
    const bool quads = width % 4 == 0 && !((uintptr_t)x & 15) && !((uintptr_t)gain & 15) && !((uintptr_t)out & 15);
#define MB_READ_NORM(T, QUADS)                                                                                                       \
    do {                                                                                                                             \
        if (smem > 48 * 1024) cudaFuncSetAttribute(hyper_read_norm_kernel<T, QUADS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        MB_LAUNCH("hyper_read_norm", (hyper_read_norm_kernel<T, QUADS>), dim3(tokens), dim3(256), smem, stream, true, x, in, gain, (T*)out, \
                  width, streams, eps);                                                                                              \
    } while (0)
    if (out_dtype == MB_F32) {
        if (quads) MB_READ_NORM(float, true); else MB_READ_NORM(float, false);
    } else if (out_dtype == MB_BF16) {
        if (quads) MB_READ_NORM(__nv_bfloat16, true); else MB_READ_NORM(__nv_bfloat16, false);
    } else {
        return fail("hyper_read_norm: unknown dtype code %d", out_dtype);
    }
#undef MB_READ_NORM
    return 0;
}

MB_EXPORT int mb_hyper_write(float* x, const void* y, int y_stride, int y_dtype, const float* out_coefficients, const float* mix,
                             int tokens, int width, int streams, cudaStream_t stream) {
    if (tokens <= 0) return 0;
    if (width <= 0 || streams <= 0 || streams > kMaxStreams) return fail("hyper_write: width %d, streams %d (at most %d)", width, streams, kMaxStreams);
    const size_t total = (size_t)tokens * width;
    const dim3 grid((unsigned)((total + 255) / 256));
    if (y_dtype == MB_F32)
        MB_LAUNCH("hyper_write", hyper_write_kernel<float>, grid, dim3(256), 0, stream, true, x, (const float*)y, y_stride, out_coefficients, mix, total, width, streams);
    else if (y_dtype == MB_BF16)
        MB_LAUNCH("hyper_write", hyper_write_kernel<__nv_bfloat16>, grid, dim3(256), 0, stream, true, x, (const __nv_bfloat16*)y, y_stride,
                  out_coefficients, mix, total, width, streams);
    else
        return fail("hyper_write: unknown dtype code %d", y_dtype);
    return 0;
}

// hyper_write of one sublayer (y float [tokens][width], row stride y_stride) and hyper_read_norm for the next, in one kernel.
MB_EXPORT int mb_hyper_write_read_norm(float* x, const float* y, int y_stride, const float* out_coefficients, const float* mix,
                                       const float* in, const float* gain, void* out, int out_dtype, int tokens, int width, int streams,
                                       float eps, cudaStream_t stream) {
    if (tokens <= 0) return 0;
    if (width <= 0 || streams <= 0 || streams > kMaxStreams) return fail("hyper_write_read_norm: width %d, streams %d (at most %d)", width, streams, kMaxStreams);
    const size_t smem = ((size_t)width + 32) * sizeof(float);
    if (smem > 200 * 1024) return fail("hyper_write_read_norm: a row of %d floats exceeds a block's shared memory", width);
    const bool quads = width % 4 == 0 && y_stride % 4 == 0 && !((uintptr_t)x & 15) && !((uintptr_t)y & 15) && !((uintptr_t)gain & 15) && !((uintptr_t)out & 15);
#define MB_WRITE_READ(T, QUADS)                                                                                                      \
    do {                                                                                                                             \
        if (smem > 48 * 1024) cudaFuncSetAttribute(hyper_write_read_norm_kernel<T, QUADS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        MB_LAUNCH("hyper_write_read_norm", (hyper_write_read_norm_kernel<T, QUADS>), dim3(tokens), dim3(256), smem, stream, true, x, y, y_stride, \
                  out_coefficients, mix, in, gain, (T*)out, width, streams, eps);                                                    \
    } while (0)
    if (out_dtype == MB_F32) {
        if (quads) MB_WRITE_READ(float, true); else MB_WRITE_READ(float, false);
    } else if (out_dtype == MB_BF16) {
        if (quads) MB_WRITE_READ(__nv_bfloat16, true); else MB_WRITE_READ(__nv_bfloat16, false);
    } else {
        return fail("hyper_write_read_norm: unknown dtype code %d", out_dtype);
    }
#undef MB_WRITE_READ
    return 0;
}
