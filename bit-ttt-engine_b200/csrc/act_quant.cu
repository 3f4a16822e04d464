// Per-token absmax int8 activation quantiser: s = max|x|/127, q = clamp(round(x*(127/max|x|))),
// round half away from zero, s == 0 -> q = 0.  The reference has no such kernel; the
// definition follows its Q8 KV-cache quantiser (layers/kv_cache.rs:95-119) without the
// zero point.  One CTA per token; x is read twice (the second pass hits L2).
#include "bt_common.cuh"

namespace bt {

template <typename T>
__device__ __forceinline__ float to_f32(T v);
template <>
__device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

__device__ __forceinline__ float block_max(float v, float* red) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    const int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = blockDim.x >> 5;
    if (l == 0) red[w] = v;
    __syncthreads();
    float r = l < nw ? red[l] : 0.0f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) r = fmaxf(r, __shfl_xor_sync(0xffffffffu, r, o));
    __syncthreads();
    return r;
}

__device__ __forceinline__ int block_sum_i32(int v, int* red) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    const int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = blockDim.x >> 5;
    if (l == 0) red[w] = v;
    __syncthreads();
    int r = l < nw ? red[l] : 0;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) r += __shfl_xor_sync(0xffffffffu, r, o);
    __syncthreads();
    return r;
}

__device__ __forceinline__ int quant_one(float x, float inv) {
    // one f32 multiply by 127/amax and round-half-away, so the CPU restatement reproduces every q
    float r = roundf(__fmul_rn(x, inv));
    r = fminf(fmaxf(r, -127.0f), 127.0f);
    return (int)r;
}

template <typename T>
__global__ void __launch_bounds__(256) act_quant_kernel(const T* __restrict__ x, int64_t k,
                                                        int8_t* __restrict__ q, int64_t q_stride,
                                                        float* __restrict__ s_out,
                                                        int32_t* __restrict__ qsum_out) {
    __shared__ float red_f[32];
    __shared__ int red_i[32];
    const int64_t row = blockIdx.x;
    const T* xr = x + row * k;
    int8_t* qr = q + row * q_stride;

    float amax = 0.0f;
    for (int64_t c = threadIdx.x; c < k; c += blockDim.x) amax = fmaxf(amax, fabsf(to_f32(xr[c])));
    amax = block_max(amax, red_f);
    const float s = __fdiv_rn(amax, 127.0f);
    const float inv = amax > 0.0f ? __fdiv_rn(127.0f, amax) : 0.0f;

    int local = 0;
    // four outputs per thread per step so that the int8 stores are 32-bit
    const int64_t k4 = k & ~(int64_t)3;
    for (int64_t c = (int64_t)threadIdx.x * 4; c < q_stride; c += (int64_t)blockDim.x * 4) {
        int v[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int64_t cc = c + j;
            v[j] = (cc < k && amax > 0.0f) ? quant_one(to_f32(xr[cc]), inv) : 0;
            local += v[j];
        }
        if (c + 3 < q_stride && ((q_stride & 3) == 0)) {
            const uint32_t packed = (uint32_t)(v[0] & 0xff) | ((uint32_t)(v[1] & 0xff) << 8) |
                                    ((uint32_t)(v[2] & 0xff) << 16) | ((uint32_t)(v[3] & 0xff) << 24);
            *reinterpret_cast<uint32_t*>(qr + c) = packed;
        } else {
#pragma unroll
            for (int j = 0; j < 4; ++j)
                if (c + j < q_stride) qr[c + j] = (int8_t)v[j];
        }
    }
    (void)k4;
    const int total = block_sum_i32(local, red_i);
    if (threadIdx.x == 0) {
        s_out[row] = s;
        if (qsum_out) qsum_out[row] = total;
    }
}

cudaError_t launch_act_quant(const void* x, bt_dtype x_dtype, int64_t m, int64_t k, int8_t* q,
                             int64_t q_stride, float* s, int32_t* qsum, cudaStream_t stream) {
    if (m <= 0) return cudaSuccess;
    if (x_dtype == BT_F32)
        act_quant_kernel<float><<<(unsigned)m, 256, 0, stream>>>((const float*)x, k, q, q_stride, s, qsum);
    else
        act_quant_kernel<__nv_bfloat16><<<(unsigned)m, 256, 0, stream>>>((const __nv_bfloat16*)x, k, q,
                                                                          q_stride, s, qsum);
    return cudaGetLastError();
}

}  // namespace bt
