// Weight-side kernels (load/export time, not on the per-step hot loop).
//
//  * pack_weight_v1      fp16 weight + per-channel scale -> the three buffers of
//                        the vdm_w4a4_packed_v1 checkpoint format, as written by
//                        weight_quantize_per_channel_kernel / pack_wscales of the
//                        reference (vdm_infer/kernels/csrc/vdm_w4a4_kernel.cu:518-551,
//                        :286-294, host side :697-728).
//  * repack_v1_to_b200   v1 packed codes -> the row-major nibble layout the
//                        tcgen05 GEMM stages with TMA (see gemm_w4a4.cuh).
//  * unswizzle_wscale_v1 v1 packed scales [N,K/64] -> plain per-channel [N].
//  * unpack_*            code extraction helpers used by the parity tests.
//
// v1 code layout (derived from the reference kernel's index arithmetic): the
// [N,K/2] byte tensor is a flat array of 16-byte entries indexed
//   [bn = n/128][bk = k/64][tile = 0..7][lane = 0..31]
// and for an entry, with n0 = bn*128 + tile*16 + lane/4 and k0 = bk*64 + (lane%4)*8,
// its four 32-bit words hold eight codes each (code e at bits [4e,4e+4)) of
//   word0: row n0,   k0..k0+7        word1: row n0,   k0+32..k0+39
//   word2: row n0+8, k0..k0+7        word3: row n0+8, k0+32..k0+39
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace b200w4a4 {
namespace detail {

// Index (in 32-bit words) of the v1 word that holds codes k8..k8+7 of row n (k8 % 8 == 0).
__host__ __device__ __forceinline__ size_t v1_word_index(int n, int k8, int K) {
  const int bn = n >> 7, r = n & 127;
  const int tile = r >> 4, rr = r & 15;
  const int hi8 = rr >> 3, lrow = rr & 7;
  const int bk = k8 >> 6, kk = k8 & 63;
  const int khalf = kk >> 5, kq = (kk & 31) >> 3;
  const int lane = lrow * 4 + kq;
  const int word = hi8 * 2 + khalf;
  return ((((static_cast<size_t>(bn) * (K >> 6) + bk) * 8 + tile) * 32 + lane) << 2) + word;
}

// Index (in halfs) of channel n's scale inside k-block bk of the v1 packed scale tensor:
// flat [bn][bk][lane][4], the four halfs of a lane being channels
// bn*128 + (lane/4)*16 + (lane%4)*2 + {0,1,8,9}.
__host__ __device__ __forceinline__ size_t v1_scale_index(int n, int bk, int K) {
  const int bn = n >> 7, r = n & 127;
  const int g = r >> 4, rr = r & 15;
  const int hi = rr >> 3, rrr = rr & 7;
  const int lane = g * 4 + (rrr >> 1);
  const int idx = hi * 2 + (rrr & 1);
  return (((static_cast<size_t>(bn) * (K >> 6) + bk) * 32 + lane) << 2) + idx;
}

__device__ __forceinline__ uint32_t weight_code(float w, float s) {
  float t = w / s;  // IEEE division; the reference multiplies by an approximate reciprocal
  t = fminf(fmaxf(t, -8.0f), 7.0f);
  return __float_as_uint(t + 12582912.0f) & 0xF;
}

}  // namespace detail

// Per-channel abs-max scale of an fp16 weight: s = amax > 0 ? fp16(amax / 7) : 1
// (token_scale_kernel applied to weight rows with clip 1, vdm_w4a4_kernel.cu:459-481, :747).
__global__ void __launch_bounds__(256)
weight_absmax_scale_kernel(const __half* __restrict__ w, __half* __restrict__ scale, int N, int K) {
  const int n = blockIdx.x;
  const __half* wr = w + static_cast<size_t>(n) * K;
  float amax = 0.0f;
  for (int k = threadIdx.x * 8; k < K; k += 256 * 8) {
    const uint4 r = *reinterpret_cast<const uint4*>(wr + k);
    const __half2* h = reinterpret_cast<const __half2*>(&r);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __half22float2(h[i]);
      amax = fmaxf(amax, fmaxf(fabsf(f.x), fabsf(f.y)));
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  __shared__ float wmax[8];
  if ((threadIdx.x & 31) == 0) wmax[threadIdx.x >> 5] = amax;
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int i = 1; i < 8; ++i) amax = fmaxf(amax, wmax[i]);
    scale[n] = amax > 0.0f ? __float2half_rn(__fdiv_rn(amax, 7.0f)) : __float2half_rn(1.0f);
  }
}

// One thread per 32-bit word of the v1 code tensor.
__global__ void __launch_bounds__(256)
pack_weight_v1_kernel(const __half* __restrict__ w, const __half* __restrict__ ch_scale,
                      uint32_t* __restrict__ packed, int N, int K) {
  const size_t j = static_cast<size_t>(blockIdx.x) * 256 + threadIdx.x;
  const size_t total = static_cast<size_t>(N) * K / 8;
  if (j >= total) return;
  const int word = static_cast<int>(j & 3);
  const int lane = static_cast<int>((j >> 2) & 31);
  const int tile = static_cast<int>((j >> 7) & 7);
  const size_t blk = j >> 10;
  const int kblocks = K >> 6;
  const int bk = static_cast<int>(blk % kblocks);
  const int bn = static_cast<int>(blk / kblocks);
  const int n = bn * 128 + tile * 16 + (lane >> 2) + (word >> 1) * 8;
  const int k = bk * 64 + (lane & 3) * 8 + (word & 1) * 32;
  const float s = __half2float(ch_scale[n]);
  const uint4 r = *reinterpret_cast<const uint4*>(w + static_cast<size_t>(n) * K + k);
  const __half2* h = reinterpret_cast<const __half2*>(&r);
  uint32_t o = 0;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __half22float2(h[i]);
    o |= detail::weight_code(f.x, s) << (8 * i);
    o |= detail::weight_code(f.y, s) << (8 * i + 4);
  }
  packed[j] = o;
}

// One thread per (channel, k-block): every k-block repeats the channel scale.
__global__ void __launch_bounds__(256)
pack_wscale_v1_kernel(const __half* __restrict__ ch_scale, __half* __restrict__ scale_packed,
                      __half* __restrict__ scale_plain, int N, int K) {
  const size_t j = static_cast<size_t>(blockIdx.x) * 256 + threadIdx.x;
  const int kblocks = K >> 6;
  if (j >= static_cast<size_t>(N) * kblocks) return;
  const int n = static_cast<int>(j / kblocks);
  const int bk = static_cast<int>(j % kblocks);
  const __half s = ch_scale[n];
  scale_packed[detail::v1_scale_index(n, bk, K)] = s;
  if (bk == 0 && scale_plain != nullptr) scale_plain[n] = s;
}

__global__ void __launch_bounds__(256)
unswizzle_wscale_v1_kernel(const __half* __restrict__ scale_packed, __half* __restrict__ scale_plain,
                           int N, int K) {
  const int n = blockIdx.x * 256 + threadIdx.x;
  if (n < N) scale_plain[n] = scale_packed[detail::v1_scale_index(n, 0, K)];
}

// One thread per 16 output bytes: row n, 32 consecutive k starting at k32.
// Output byte i holds code[k32+i] in the high nibble and code[k32+16+i] in the low nibble.
__global__ void __launch_bounds__(256)
repack_v1_to_b200_kernel(const uint32_t* __restrict__ v1, uint4* __restrict__ out, int N, int K) {
  const size_t j = static_cast<size_t>(blockIdx.x) * 256 + threadIdx.x;
  const int chunks_per_row = K >> 5;
  if (j >= static_cast<size_t>(N) * chunks_per_row) return;
  const int n = static_cast<int>(j / chunks_per_row);
  const int k32 = static_cast<int>(j % chunks_per_row) << 5;
  const uint32_t h0 = v1[detail::v1_word_index(n, k32, K)];
  const uint32_t h1 = v1[detail::v1_word_index(n, k32 + 8, K)];
  const uint32_t l0 = v1[detail::v1_word_index(n, k32 + 16, K)];
  const uint32_t l1 = v1[detail::v1_word_index(n, k32 + 24, K)];
  auto weave = [](uint32_t hi, uint32_t lo, int first) {
    uint32_t o = 0;
#pragma unroll
    for (int b = 0; b < 4; ++b) {
      const uint32_t hn = (hi >> (4 * (first + b))) & 0xF;
      const uint32_t ln = (lo >> (4 * (first + b))) & 0xF;
      o |= ((hn << 4) | ln) << (8 * b);
    }
    return o;
  };
  uint4 o;
  o.x = weave(h0, l0, 0);
  o.y = weave(h0, l0, 4);
  o.z = weave(h1, l1, 0);
  o.w = weave(h1, l1, 4);
  out[j] = o;
}

// Load-time expansion for the int8-staged GEMM variant: v1 codes -> row-major int8 [N,K] with every
// byte equal to 16 * code (the value the unpack warps would otherwise produce in shared memory).
// One thread per 8 consecutive k of a row (one v1 word in, 8 bytes out).
__global__ void __launch_bounds__(256)
expand_v1_to_int8_kernel(const uint32_t* __restrict__ v1, uint2* __restrict__ out, int N, int K) {
  const size_t j = static_cast<size_t>(blockIdx.x) * 256 + threadIdx.x;
  const int words_per_row = K >> 3;
  if (j >= static_cast<size_t>(N) * words_per_row) return;
  const int n = static_cast<int>(j / words_per_row);
  const int k8 = static_cast<int>(j % words_per_row) << 3;
  const uint32_t wv = v1[detail::v1_word_index(n, k8, K)];
  uint2 o;
  o.x = ((wv & 0xFu) << 4) | ((wv & 0xF0u) << 8) | ((wv & 0xF00u) << 12) | ((wv & 0xF000u) << 16);
  const uint32_t hi = wv >> 16;
  o.y = ((hi & 0xFu) << 4) | ((hi & 0xF0u) << 8) | ((hi & 0xF00u) << 12) | ((hi & 0xF000u) << 16);
  out[j] = o;
}

// ---- test helpers: extract int8 codes [rows,K] ---------------------------------
__global__ void __launch_bounds__(256)
unpack_int8_weight_kernel(const int8_t* __restrict__ w8, int8_t* __restrict__ codes, int N, int K) {
  const size_t j = static_cast<size_t>(blockIdx.x) * 256 + threadIdx.x;
  if (j >= static_cast<size_t>(N) * K) return;
  codes[j] = static_cast<int8_t>(w8[j] >> 4);   // arithmetic shift: exact, every byte is 16 * code
}

__global__ void __launch_bounds__(256)
unpack_b200_weight_kernel(const uint8_t* __restrict__ wr, int8_t* __restrict__ codes, int N, int K) {
  const size_t j = static_cast<size_t>(blockIdx.x) * 256 + threadIdx.x;
  if (j >= static_cast<size_t>(N) * K) return;
  const int n = static_cast<int>(j / K), k = static_cast<int>(j % K);
  const int kin = k & 31;
  const uint8_t b = wr[static_cast<size_t>(n) * (K / 2) + (k >> 5) * 16 + (kin & 15)];
  const int nib = (kin < 16) ? (b >> 4) : (b & 0xF);
  codes[j] = static_cast<int8_t>((nib ^ 8) - 8);
}

__global__ void __launch_bounds__(256)
unpack_v1_weight_kernel(const uint32_t* __restrict__ v1, int8_t* __restrict__ codes, int N, int K) {
  const size_t j = static_cast<size_t>(blockIdx.x) * 256 + threadIdx.x;
  if (j >= static_cast<size_t>(N) * K) return;
  const int n = static_cast<int>(j / K), k = static_cast<int>(j % K);
  const uint32_t wv = v1[detail::v1_word_index(n, k & ~7, K)];
  const int nib = (wv >> (4 * (k & 7))) & 0xF;
  codes[j] = static_cast<int8_t>((nib ^ 8) - 8);
}

__global__ void __launch_bounds__(256)
unpack_nibble_rows_kernel(const uint8_t* __restrict__ q, int8_t* __restrict__ codes, int M, int K) {
  const size_t j = static_cast<size_t>(blockIdx.x) * 256 + threadIdx.x;
  if (j >= static_cast<size_t>(M) * K) return;
  const uint8_t b = q[j >> 1];
  const int nib = (j & 1) ? (b >> 4) : (b & 0xF);
  codes[j] = static_cast<int8_t>((nib ^ 8) - 8);
}

}  // namespace b200w4a4
