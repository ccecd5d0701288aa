// Per-tensor e4m3 quantisation helper used to prepare fp8 GEMM operands:
//   scale = max|x| / 448,   y = e4m3_rn(x / scale).
// Two launches: a grid-stride abs-max reduction (warp shuffle, then one atomicMax on the bit
// pattern of the non-negative float per block) and the cast.  HBM-bound: reads x twice (8 B per
// element) and writes 1 B per element.
#include <cuda_fp8.h>

#include "common.cuh"

namespace b200k {
namespace {

constexpr float kE4M3Max = 448.0f;

__global__ void absmax_kernel(const float* __restrict__ x, int64_t n, uint32_t* __restrict__ amax_bits) {
  float m = 0.f;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  const int64_t n4 = n / 4;
  const float4* x4 = reinterpret_cast<const float4*>(x);
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n4; i += stride) {
    const float4 v = __ldg(x4 + i);
    m = fmaxf(m, fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))));
  }
  for (int64_t i = n4 * 4 + static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride)
    m = fmaxf(m, fabsf(x[i]));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  __shared__ float wm[32];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) wm[warp] = m;
  __syncthreads();
  if (warp == 0) {
    m = lane < (blockDim.x >> 5) ? wm[lane] : 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    if (lane == 0) atomicMax(amax_bits, __float_as_uint(m));  // non-negative floats order like their bits
  }
}

__global__ void cast_e4m3_kernel(const float* __restrict__ x, uint8_t* __restrict__ y, int64_t n,
                                 const uint32_t* __restrict__ amax_bits, float* __restrict__ scale_out) {
  const float amax = __uint_as_float(*amax_bits);
  const float scale = amax > 0.f ? __fdiv_rn(amax, kE4M3Max) : 1.0f;
  if (blockIdx.x == 0 && threadIdx.x == 0) *scale_out = scale;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  const int64_t n4 = n / 4;
  const float4* x4 = reinterpret_cast<const float4*>(x);
  uint32_t* y4 = reinterpret_cast<uint32_t*>(y);
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n4; i += stride) {
    const float4 v = __ldg(x4 + i);
    const uint32_t b0 = __nv_cvt_float_to_fp8(__fdiv_rn(v.x, scale), __NV_SATFINITE, __NV_E4M3);
    const uint32_t b1 = __nv_cvt_float_to_fp8(__fdiv_rn(v.y, scale), __NV_SATFINITE, __NV_E4M3);
    const uint32_t b2 = __nv_cvt_float_to_fp8(__fdiv_rn(v.z, scale), __NV_SATFINITE, __NV_E4M3);
    const uint32_t b3 = __nv_cvt_float_to_fp8(__fdiv_rn(v.w, scale), __NV_SATFINITE, __NV_E4M3);
    y4[i] = b0 | (b1 << 8) | (b2 << 16) | (b3 << 24);
  }
  for (int64_t i = n4 * 4 + static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride)
    y[i] = __nv_cvt_float_to_fp8(__fdiv_rn(x[i], scale), __NV_SATFINITE, __NV_E4M3);
}

}  // namespace

int launch_quantize_e4m3(const float* x, void* y, float* scale_out, uint32_t* amax_scratch, int64_t n,
                         cudaStream_t stream) {
  if (!x || !y || !scale_out || !amax_scratch) return set_error(B200K_ERR_NULL, "quantize_e4m3: NULL pointer");
  if (n <= 0) return set_error(B200K_ERR_BAD_SHAPE, "quantize_e4m3: n must be positive");
  if ((reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(y) & 3))
    return set_error(B200K_ERR_BAD_ALIGN, "quantize_e4m3: x must be 16-byte aligned and y 4-byte aligned");
  int rc = ensure_sm100();
  if (rc) return rc;
  rc = check_cuda(cudaMemsetAsync(amax_scratch, 0, sizeof(uint32_t), stream), "quantize_e4m3: memset");
  if (rc) return rc;
  const int threads = 256;
  int64_t want = (n / 4 + threads - 1) / threads;
  const int64_t cap = static_cast<int64_t>(num_sms()) * 8;
  const int blocks = static_cast<int>(want < 1 ? 1 : (want > cap ? cap : want));
  absmax_kernel<<<blocks, threads, 0, stream>>>(x, n, amax_scratch);
  rc = check_cuda(cudaGetLastError(), "absmax_kernel launch");
  if (rc) return rc;
  cast_e4m3_kernel<<<blocks, threads, 0, stream>>>(x, reinterpret_cast<uint8_t*>(y), n, amax_scratch, scale_out);
  return check_cuda(cudaGetLastError(), "cast_e4m3_kernel launch");
}

}  // namespace b200k
