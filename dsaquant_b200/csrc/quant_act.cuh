// Dynamic per-token symmetric int4 activation quantiser: one pass over x.
//
// Replaces token_scale_kernel + act_quantize_per_token_kernel of the reference
// (vdm_infer/kernels/csrc/vdm_w4a4_kernel.cu:459-481 and :483-516), which read
// every row twice (abs-max pass, then quantise pass) with one-warp CTAs.  Here
// a row is loaded once with 128-bit requests, kept in registers across the
// abs-max reduction (warp shuffles, plus a shared-memory hop when a row spans
// several warps) and written back as codes with coalesced vector stores.
//
// Pinned arithmetic (IEEE fp32, no fast-math):
//   amax  = max_k |x[m,k]|
//   s[m]  = (max(amax, 1e-5f) / 7.0f) * clip
//   q     = clamp(rint(x / s[m]), -8, 7)            (true division, ties to even)
// which is UniformQuantizer's symmetric path on an fp32 2-D input
// (vdm_infer/quantization/quant_linear.py:43-48, :64-66) with the clip applied
// to the scale as the kernel path does (vdm_w4a4_kernel.cu:478).
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace b200w4a4 {

enum : int { XDT_F16 = 0, XDT_BF16 = 1, XDT_F32 = 2 };
// Output container of the codes.
enum : int {
  QOUT_INT8 = 0,    // int8 [M,K], one code per byte: what the GEMM's TMA loads
  QOUT_NIBBLE = 1,  // u8 [M,K/2], element 2b in the low nibble, 2b+1 in the high nibble
};

namespace detail {

template <typename T>
__device__ __forceinline__ void load8(const T* p, float (&v)[8]);

template <>
__device__ __forceinline__ void load8<__half>(const __half* p, float (&v)[8]) {
  const uint4 r = __ldcs(reinterpret_cast<const uint4*>(p));
  const __half2* h = reinterpret_cast<const __half2*>(&r);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __half22float2(h[i]);
    v[2 * i] = f.x;
    v[2 * i + 1] = f.y;
  }
}
template <>
__device__ __forceinline__ void load8<__nv_bfloat16>(const __nv_bfloat16* p, float (&v)[8]) {
  const uint4 r = __ldcs(reinterpret_cast<const uint4*>(p));
  const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    v[2 * i] = __uint_as_float(w[i] << 16);
    v[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
  }
}
template <>
__device__ __forceinline__ void load8<float>(const float* p, float (&v)[8]) {
  const float4 a = __ldcs(reinterpret_cast<const float4*>(p));
  const float4 b = __ldcs(reinterpret_cast<const float4*>(p) + 1);
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
  v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}

// clamp(rint(x / s), -8, 7) as the low byte of the result (two's complement).
// Clamping first is equivalent because the bounds are integers; adding
// 1.5 * 2^23 rounds to nearest-even and leaves the integer in the low mantissa bits.
__device__ __forceinline__ uint32_t code_bits(float x, float s) {
  float t = x / s;
  t = fminf(fmaxf(t, -8.0f), 7.0f);
  return __float_as_uint(t + 12582912.0f);
}

__device__ __forceinline__ float row_scale(float amax, float clip) {
  return __fmul_rn(__fdiv_rn(fmaxf(amax, 1e-5f), 7.0f), clip);
}

template <int QOUT>
__device__ __forceinline__ void store8(void* q, size_t row, int K, int chunk, const float (&v)[8],
                                       float s) {
  uint32_t c[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) c[i] = code_bits(v[i], s);
  if constexpr (QOUT == QOUT_INT8) {
    uint2 o;
    o.x = (c[0] & 0xFF) | ((c[1] & 0xFF) << 8) | ((c[2] & 0xFF) << 16) | (c[3] << 24);
    o.y = (c[4] & 0xFF) | ((c[5] & 0xFF) << 8) | ((c[6] & 0xFF) << 16) | (c[7] << 24);
    *reinterpret_cast<uint2*>(static_cast<uint8_t*>(q) + row * K + 8 * static_cast<size_t>(chunk)) = o;
  } else {
    uint32_t o = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) o |= (c[i] & 0xF) << (4 * i);
    *reinterpret_cast<uint32_t*>(static_cast<uint8_t*>(q) + row * (K / 2) +
                                 4 * static_cast<size_t>(chunk)) = o;
  }
}

}  // namespace detail

// TPR threads cooperate on one row and each holds up to NCH chunks of 8 values.
template <typename T, int TPR, int NCH, int QOUT>
__global__ void __launch_bounds__(256)
quant_act_rows_kernel(const T* __restrict__ x, void* __restrict__ q, float* __restrict__ scale,
                      int M, int K, float clip) {
  constexpr int ROWS = 256 / TPR;
  const int sub = threadIdx.x / TPR;
  const int t = threadIdx.x % TPR;
  const long long row = static_cast<long long>(blockIdx.x) * ROWS + sub;
  const bool row_ok = row < M;
  const int nchunks = K >> 3;
  const T* xr = x + (row_ok ? row : 0) * static_cast<long long>(K);

  float v[NCH][8];
  float amax = 0.0f;
#pragma unroll
  for (int i = 0; i < NCH; ++i) {
    const int c = t + i * TPR;
    if (row_ok && c < nchunks) {
      detail::load8<T>(xr + 8 * c, v[i]);
#pragma unroll
      for (int e = 0; e < 8; ++e) amax = fmaxf(amax, fabsf(v[i][e]));
    }
  }
  constexpr int W = TPR < 32 ? TPR : 32;
#pragma unroll
  for (int o = W / 2; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  if constexpr (TPR > 32) {
    __shared__ float wmax[8];
    const int warp = threadIdx.x >> 5;
    if ((threadIdx.x & 31) == 0) wmax[warp] = amax;
    __syncthreads();
    constexpr int WPR = TPR / 32;
    const int w0 = sub * WPR;
    amax = wmax[w0];
#pragma unroll
    for (int w = 1; w < WPR; ++w) amax = fmaxf(amax, wmax[w0 + w]);
  }
  const float s = detail::row_scale(amax, clip);
  if (!row_ok) return;
  if (t == 0) scale[row] = s;
#pragma unroll
  for (int i = 0; i < NCH; ++i) {
    const int c = t + i * TPR;
    if (c < nchunks) detail::store8<QOUT>(q, static_cast<size_t>(row), K, c, v[i], s);
  }
}

// Rows too long to hold in registers: one CTA per row, two passes (the second
// pass re-reads the row, which was just touched and sits in L1/L2).
template <typename T, int QOUT>
__global__ void __launch_bounds__(256)
quant_act_long_rows_kernel(const T* __restrict__ x, void* __restrict__ q,
                           float* __restrict__ scale, int M, int K, float clip) {
  const long long row = blockIdx.x;
  const int nchunks = K >> 3;
  const T* xr = x + row * static_cast<long long>(K);
  float amax = 0.0f;
  for (int c = threadIdx.x; c < nchunks; c += 256) {
    float v[8];
    detail::load8<T>(xr + 8 * c, v);
#pragma unroll
    for (int e = 0; e < 8; ++e) amax = fmaxf(amax, fabsf(v[e]));
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  __shared__ float wmax[8];
  if ((threadIdx.x & 31) == 0) wmax[threadIdx.x >> 5] = amax;
  __syncthreads();
  amax = wmax[0];
#pragma unroll
  for (int w = 1; w < 8; ++w) amax = fmaxf(amax, wmax[w]);
  const float s = detail::row_scale(amax, clip);
  if (threadIdx.x == 0) scale[row] = s;
  for (int c = threadIdx.x; c < nchunks; c += 256) {
    float v[8];
    detail::load8<T>(xr + 8 * c, v);
    detail::store8<QOUT>(q, static_cast<size_t>(row), K, c, v, s);
  }
}

template <typename T, int QOUT>
inline cudaError_t launch_quant_act(const T* x, void* q, float* scale, int M, int K, float clip,
                                    cudaStream_t stream) {
  const int nchunks = K / 8;
#define B200W4A4_QLAUNCH(TPR, NCH)                                                            \
  do {                                                                                         \
    constexpr int ROWS = 256 / (TPR);                                                          \
    const unsigned grid = static_cast<unsigned>((static_cast<long long>(M) + ROWS - 1) / ROWS); \
    quant_act_rows_kernel<T, TPR, NCH, QOUT><<<grid, 256, 0, stream>>>(x, q, scale, M, K, clip); \
  } while (0)
  if (nchunks <= 32 * 4) B200W4A4_QLAUNCH(32, 4);
  else if (nchunks <= 32 * 8) B200W4A4_QLAUNCH(32, 8);
  else if (nchunks <= 64 * 8) B200W4A4_QLAUNCH(64, 8);
  else if (nchunks <= 128 * 4) B200W4A4_QLAUNCH(128, 4);
  else if (nchunks <= 128 * 8) B200W4A4_QLAUNCH(128, 8);
  else if (nchunks <= 256 * 4) B200W4A4_QLAUNCH(256, 4);
  else if (nchunks <= 256 * 8) B200W4A4_QLAUNCH(256, 8);
  else
    quant_act_long_rows_kernel<T, QOUT><<<static_cast<unsigned>(M), 256, 0, stream>>>(x, q, scale, M,
                                                                                      K, clip);
#undef B200W4A4_QLAUNCH
  return cudaGetLastError();
}

}  // namespace b200w4a4
