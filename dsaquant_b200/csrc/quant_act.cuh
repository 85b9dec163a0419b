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
// The kernel evaluates q with two fused multiply-adds per value and falls back to the division
// for values near a rounding tie, which provably yields the same integer (see chunk_codes).
// This is UniformQuantizer's symmetric path on an fp32 2-D input
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

// Work fused in front of the quantiser (what the caller would otherwise run as separate
// elementwise / normalisation kernels over the same rows).
enum : int {
  PRE_NONE = 0,
  PRE_GELU_TANH = 1,      // v = fp16(gelu_tanh(x))                       (FFN: between up and down projection)
  PRE_LAYERNORM_MOD = 2,  // v = fp16(fp16(layernorm(x)) * (1 + scale[k]) + shift[k])   (block entry modulation)
};

struct PreArgs {
  const float* mod_scale;    // [K] (or [M,K] with mod_row_stride = K)
  const float* mod_shift;
  long long mod_row_stride;  // 0: one vector for every row
  float ln_eps;
};

namespace detail {

// tanh-GELU evaluated in fp32 with the constants and operation order of the usual
// "gelu(approximate='tanh')" definition; the caller rounds to fp16 like the tensor it replaces.
__device__ __forceinline__ float gelu_tanh_f32(float x) {
  const float kBeta = 0.7978845608028654f;  // sqrt(2/pi)
  const float kKappa = 0.044715f;
  const float x3 = x * x * x;
  const float inner = kBeta * (x + kKappa * x3);
  return 0.5f * x * (1.0f + tanhf(inner));
}

// A chunk is 8 consecutive values of a row, kept in registers in its storage format.
template <typename T>
struct Chunk;

template <>
struct Chunk<__half> {
  uint4 raw;
  __device__ __forceinline__ void load(const __half* p) { raw = __ldcs(reinterpret_cast<const uint4*>(p)); }
  // max |v| over the chunk, folded into a running packed maximum (no conversion needed:
  // the maximum of fp16 values is one of them).
  __device__ __forceinline__ void absmax(float& m) const {
    const __half2* h = reinterpret_cast<const __half2*>(&raw);
    __half2 a = __hmax2(__habs2(h[0]), __habs2(h[1]));
    __half2 b = __hmax2(__habs2(h[2]), __habs2(h[3]));
    a = __hmax2(a, b);
    m = fmaxf(m, fmaxf(__low2float(a), __high2float(a)));
  }
  __device__ __forceinline__ void values(float (&v)[8]) const {
    const __half2* h = reinterpret_cast<const __half2*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __half22float2(h[i]);
      v[2 * i] = f.x;
      v[2 * i + 1] = f.y;
    }
  }
};

template <>
struct Chunk<__nv_bfloat16> {
  uint4 raw;
  __device__ __forceinline__ void load(const __nv_bfloat16* p) {
    raw = __ldcs(reinterpret_cast<const uint4*>(p));
  }
  __device__ __forceinline__ void values(float (&v)[8]) const {
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      v[2 * i] = __uint_as_float(w[i] << 16);
      v[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
    }
  }
  // packed maxima, as for fp16: the maximum of bf16 values is one of them
  __device__ __forceinline__ void absmax(float& m) const {
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
    __nv_bfloat162 a = __hmax2(__habs2(h[0]), __habs2(h[1]));
    __nv_bfloat162 b = __hmax2(__habs2(h[2]), __habs2(h[3]));
    a = __hmax2(a, b);
    m = fmaxf(m, fmaxf(__low2float(a), __high2float(a)));
  }
};

template <>
struct Chunk<float> {
  float4 lo, hi;
  __device__ __forceinline__ void load(const float* p) {
    lo = __ldcs(reinterpret_cast<const float4*>(p));
    hi = __ldcs(reinterpret_cast<const float4*>(p) + 1);
  }
  __device__ __forceinline__ void values(float (&v)[8]) const {
    v[0] = lo.x; v[1] = lo.y; v[2] = lo.z; v[3] = lo.w;
    v[4] = hi.x; v[5] = hi.y; v[6] = hi.z; v[7] = hi.w;
  }
  __device__ __forceinline__ void absmax(float& m) const {
    float v[8];
    values(v);
#pragma unroll
    for (int e = 0; e < 8; ++e) m = fmaxf(m, fabsf(v[e]));
  }
};

constexpr float kRoundMagic = 12582912.0f;  // 1.5 * 2^23: adding it rounds to nearest-even

__device__ __forceinline__ float row_scale(float amax, float clip) {
  return __fmul_rn(__fdiv_rn(fmaxf(amax, 1e-5f), 7.0f), clip);
}

// Bits of (clamp(rint(x / s), -8, 7) + magic): the code is the low byte (two's complement).
// Clamping first is equivalent because the bounds are integers.
__device__ __forceinline__ uint32_t code_bits_div(float x, float s) {
  float t = __fdiv_rn(x, s);
  t = fminf(fmaxf(t, -8.0f), 7.0f);
  return __float_as_uint(t + kRoundMagic);
}

// Per-row constants of the fast path.
struct RowQuant {
  float s;          // scale
  float r_up, r_dn; // RN(1/s) nudged up / down by 2^-20: brackets of the true reciprocal
  bool exact_only;  // scale so large or small that 1/s is not a normal number: always divide
  bool clamp;       // |x/s| can exceed 7.5 (clip below ~0.934): clamp the rounded values
};

// Eight codes of one chunk.  Fast path: two fused multiply-adds per value,
//   ya = RN(x * r_up + magic),  yb = RN(x * r_dn + magic),
// each a single rounding of the exact product to an integer (ties to even, like rint).  The
// products bracket both the true quotient and its fp32 rounding fl(x/s), because r_up / r_dn
// differ from 1/s by at least 2^-21 relative while RN(1/s) and fl(x/s) are off by at most 2^-24
// each; rint is monotonic, so ya == yb implies rint(fl(x/s)) == ya.  When they differ somewhere
// in the chunk (a value within ~2^-16 of a rounding tie: a few chunks per hundred thousand) the
// chunk is redone with the IEEE division, so the result equals clamp(rint(x / s)) for every input.
template <bool CLAMP>
__device__ __forceinline__ uint32_t chunk_codes_fast(const float (&v)[8], const RowQuant& rq, uint32_t (&c)[8]) {
  uint32_t diff = 0;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    float ya = __fmaf_rn(v[i], rq.r_up, kRoundMagic);
    float yb = __fmaf_rn(v[i], rq.r_dn, kRoundMagic);
    if constexpr (CLAMP) {
      ya = fminf(fmaxf(ya, kRoundMagic - 8.0f), kRoundMagic + 7.0f);
      yb = fminf(fmaxf(yb, kRoundMagic - 8.0f), kRoundMagic + 7.0f);
    }
    diff |= __float_as_uint(ya) ^ __float_as_uint(yb);
    c[i] = __float_as_uint(ya);
  }
  return diff;
}

__device__ __forceinline__ void chunk_codes(const float (&v)[8], const RowQuant& rq, uint32_t (&c)[8]) {
  // rq.clamp is the same for the whole launch: two straight-line bodies, one uniform branch.
  const uint32_t diff = rq.clamp ? chunk_codes_fast<true>(v, rq, c) : chunk_codes_fast<false>(v, rq, c);
  if (rq.exact_only || diff != 0) {
#pragma unroll
    for (int i = 0; i < 8; ++i) c[i] = code_bits_div(v[i], rq.s);
  }
}

template <int QOUT>
__device__ __forceinline__ void store_codes(void* q, size_t row, int K, int chunk,
                                            const uint32_t (&c)[8]) {
  if constexpr (QOUT == QOUT_INT8) {
    uint2 o;
    o.x = __byte_perm(__byte_perm(c[0], c[1], 0x0040), __byte_perm(c[2], c[3], 0x0040), 0x5410);
    o.y = __byte_perm(__byte_perm(c[4], c[5], 0x0040), __byte_perm(c[6], c[7], 0x0040), 0x5410);
    *reinterpret_cast<uint2*>(static_cast<uint8_t*>(q) + row * K + 8 * static_cast<size_t>(chunk)) = o;
  } else {
    uint32_t o = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) o |= (c[i] & 0xF) << (4 * i);
    *reinterpret_cast<uint32_t*>(static_cast<uint8_t*>(q) + row * (K / 2) +
                                 4 * static_cast<size_t>(chunk)) = o;
  }
}

__device__ __forceinline__ RowQuant row_quant(float amax, float clip) {
  RowQuant rq;
  rq.s = row_scale(amax, clip);
  rq.exact_only = !(rq.s < 1.0e30f) || !(rq.s > 1.0e-30f);  // also true for NaN / inf scales
  const float r = rq.exact_only ? 0.0f : __frcp_rn(rq.s);
  rq.r_up = __fmul_rn(r, 1.0f + 9.5367431640625e-07f);  // 1 + 2^-20
  rq.r_dn = __fmul_rn(r, 1.0f - 9.5367431640625e-07f);
  // |x| <= amax gives |x/s| <= 7/clip; rounding stays within [-7, 7] while that is below 7.5.
  rq.clamp = !(clip >= 0.934f);
  return rq;
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

  detail::Chunk<T> ch[NCH];
  float amax = 0.0f;
#pragma unroll
  for (int i = 0; i < NCH; ++i) {
    const int c = t + i * TPR;
    if (row_ok && c < nchunks) ch[i].load(xr + 8 * c);
  }
#pragma unroll
  for (int i = 0; i < NCH; ++i) {
    const int c = t + i * TPR;
    if (row_ok && c < nchunks) ch[i].absmax(amax);
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
  if (!row_ok) return;
  const detail::RowQuant rq = detail::row_quant(amax, clip);
  if (t == 0) scale[row] = rq.s;
#pragma unroll
  for (int i = 0; i < NCH; ++i) {
    const int c = t + i * TPR;
    if (c < nchunks) {
      float v[8];
      uint32_t codes[8];
      ch[i].values(v);
      detail::chunk_codes(v, rq, codes);
      detail::store_codes<QOUT>(q, static_cast<size_t>(row), K, c, codes);
    }
  }
}

// Reduction of one value over the TPR threads that share a row (sum or max).
template <int TPR, bool IS_MAX>
__device__ __forceinline__ float row_reduce(float v, float* smem8, int sub) {
  constexpr int W = TPR < 32 ? TPR : 32;
#pragma unroll
  for (int o = W / 2; o > 0; o >>= 1) {
    const float other = __shfl_xor_sync(0xffffffffu, v, o);
    v = IS_MAX ? fmaxf(v, other) : v + other;
  }
  if constexpr (TPR > 32) {
    const int warp = threadIdx.x >> 5;
    if ((threadIdx.x & 31) == 0) smem8[warp] = v;
    __syncthreads();
    constexpr int WPR = TPR / 32;
    const int w0 = sub * WPR;
    v = smem8[w0];
#pragma unroll
    for (int w = 1; w < WPR; ++w) v = IS_MAX ? fmaxf(v, smem8[w0 + w]) : v + smem8[w0 + w];
  }
  return v;
}

// Quantiser with a fused prologue (fp16 input, int8 container).  The row stays in registers
// across the prologue's own reductions (mean, variance) and the abs-max, so x is still read once
// and the normalised / activated tensor is never written to memory.
template <int TPR, int NCH, int PRE>
__global__ void __launch_bounds__(256)
quant_act_pre_rows_kernel(const __half* __restrict__ x, void* __restrict__ q,
                          float* __restrict__ scale, int M, int K, float clip, PreArgs pre) {
  constexpr int ROWS = 256 / TPR;
  __shared__ float red[3][8];
  const int sub = threadIdx.x / TPR;
  const int t = threadIdx.x % TPR;
  const long long row = static_cast<long long>(blockIdx.x) * ROWS + sub;
  const bool row_ok = row < M;
  const int nchunks = K >> 3;
  const __half* xr = x + (row_ok ? row : 0) * static_cast<long long>(K);

  detail::Chunk<__half> ch[NCH];
#pragma unroll
  for (int i = 0; i < NCH; ++i) {
    const int c = t + i * TPR;
    if (row_ok && c < nchunks) ch[i].load(xr + 8 * c);
  }

  float mean = 0.0f, rstd = 1.0f;
  if constexpr (PRE == PRE_LAYERNORM_MOD) {
    float sum = 0.0f;
#pragma unroll
    for (int i = 0; i < NCH; ++i) {
      const int c = t + i * TPR;
      if (row_ok && c < nchunks) {
        float v[8];
        ch[i].values(v);
#pragma unroll
        for (int e = 0; e < 8; ++e) sum += v[e];
      }
    }
    mean = row_reduce<TPR, false>(sum, red[0], sub) / static_cast<float>(K);
    float sq = 0.0f;
#pragma unroll
    for (int i = 0; i < NCH; ++i) {
      const int c = t + i * TPR;
      if (row_ok && c < nchunks) {
        float v[8];
        ch[i].values(v);
#pragma unroll
        for (int e = 0; e < 8; ++e) sq += (v[e] - mean) * (v[e] - mean);
      }
    }
    const float var = row_reduce<TPR, false>(sq, red[1], sub) / static_cast<float>(K);
    rstd = rsqrtf(var + pre.ln_eps);
  }

  // The prologue's output for chunk i in fp32, before its final rounding to fp16 (done once, by the
  // packing conversion below).
  auto transformed = [&](int i, int c, float (&v)[8]) {
    ch[i].values(v);
    if constexpr (PRE == PRE_GELU_TANH) {
#pragma unroll
      for (int e = 0; e < 8; ++e) v[e] = detail::gelu_tanh_f32(v[e]);
    } else if constexpr (PRE == PRE_LAYERNORM_MOD) {
      const float* ms = pre.mod_scale + row * pre.mod_row_stride + 8 * c;
      const float* mh = pre.mod_shift + row * pre.mod_row_stride + 8 * c;
      const float4 s0 = __ldg(reinterpret_cast<const float4*>(ms)), s1 = __ldg(reinterpret_cast<const float4*>(ms) + 1);
      const float4 h0 = __ldg(reinterpret_cast<const float4*>(mh)), h1 = __ldg(reinterpret_cast<const float4*>(mh) + 1);
      const float sc[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
      const float sh[8] = {h0.x, h0.y, h0.z, h0.w, h1.x, h1.y, h1.z, h1.w};
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const float n16 = __half2float(__float2half_rn((v[e] - mean) * rstd));   // layer norm, cast to fp16
        v[e] = __fadd_rn(__fmul_rn(n16, __fadd_rn(1.0f, sc[e])), sh[e]);          // * (1 + scale) + shift
      }
    }
  };

  // The prologue's output is fp16 by definition, so it replaces the raw chunk in registers: the
  // modulation vectors are read (and tanh evaluated) once, and the abs-max and the codes below
  // work on the stored fp16 values exactly as the plain kernel does.
  float amax = 0.0f;
#pragma unroll
  for (int i = 0; i < NCH; ++i) {
    const int c = t + i * TPR;
    if (row_ok && c < nchunks) {
      float v[8];
      transformed(i, c, v);
      __half2 h[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) h[e] = __floats2half2_rn(v[2 * e], v[2 * e + 1]);  // the prologue's one rounding to fp16
      ch[i].raw = *reinterpret_cast<const uint4*>(h);
      ch[i].absmax(amax);
    }
  }
  amax = row_reduce<TPR, true>(amax, red[2], sub);
  if (!row_ok) return;
  const detail::RowQuant rq = detail::row_quant(amax, clip);
  if (t == 0) scale[row] = rq.s;
#pragma unroll
  for (int i = 0; i < NCH; ++i) {
    const int c = t + i * TPR;
    if (c < nchunks) {
      float v[8];
      uint32_t codes[8];
      ch[i].values(v);
      detail::chunk_codes(v, rq, codes);
      detail::store_codes<QOUT_INT8>(q, static_cast<size_t>(row), K, c, codes);
    }
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
    detail::Chunk<T> ch;
    ch.load(xr + 8 * c);
    ch.absmax(amax);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  __shared__ float wmax[8];
  if ((threadIdx.x & 31) == 0) wmax[threadIdx.x >> 5] = amax;
  __syncthreads();
  amax = wmax[0];
#pragma unroll
  for (int w = 1; w < 8; ++w) amax = fmaxf(amax, wmax[w]);
  const detail::RowQuant rq = detail::row_quant(amax, clip);
  if (threadIdx.x == 0) scale[row] = rq.s;
  for (int c = threadIdx.x; c < nchunks; c += 256) {
    detail::Chunk<T> ch;
    float v[8];
    uint32_t codes[8];
    ch.load(xr + 8 * c);
    ch.values(v);
    detail::chunk_codes(v, rq, codes);
    detail::store_codes<QOUT>(q, static_cast<size_t>(row), K, c, codes);
  }
}

template <typename T, int QOUT>
inline cudaError_t launch_quant_act(const T* x, void* q, float* scale, int M, int K, float clip,
                                    cudaStream_t stream) {
  const int nchunks = K / 8;
  // One-shot CTAs, several resident per SM: measured faster than a persistent variant that
  // prefetches the next row into a second register set (fewer resident warps cost more than the
  // prefetch gained: 4.8 vs 6.1 TB/s at K = 5120).
#define B200W4A4_QLAUNCH(TPR, NCH)                                                            \
  do {                                                                                         \
    constexpr int ROWS = 256 / (TPR);                                                          \
    const unsigned grid = static_cast<unsigned>((static_cast<long long>(M) + ROWS - 1) / ROWS); \
    quant_act_rows_kernel<T, TPR, NCH, QOUT><<<grid, 256, 0, stream>>>(x, q, scale, M, K, clip); \
  } while (0)
  if (nchunks <= 32 * 4) B200W4A4_QLAUNCH(32, 4);
  else if (nchunks <= 32 * 6) B200W4A4_QLAUNCH(32, 6);    // K = 1536
  else if (nchunks <= 32 * 8) B200W4A4_QLAUNCH(32, 8);
  else if (nchunks <= 64 * 6) B200W4A4_QLAUNCH(64, 6);    // K = 3072
  else if (nchunks <= 64 * 8) B200W4A4_QLAUNCH(64, 8);
  else if (nchunks <= 128 * 4) B200W4A4_QLAUNCH(128, 4);
  else if (nchunks <= 128 * 5) B200W4A4_QLAUNCH(128, 5);  // K = 5120
  else if (nchunks <= 128 * 8) B200W4A4_QLAUNCH(128, 8);
  else if (nchunks <= 256 * 4) B200W4A4_QLAUNCH(256, 4);
  else if (nchunks <= 256 * 5) B200W4A4_QLAUNCH(256, 5);  // K = 8960
  else if (nchunks <= 256 * 7) B200W4A4_QLAUNCH(256, 7);  // K = 13824, 14336
  else if (nchunks <= 256 * 8) B200W4A4_QLAUNCH(256, 8);
  else
    quant_act_long_rows_kernel<T, QOUT><<<static_cast<unsigned>(M), 256, 0, stream>>>(x, q, scale, M,
                                                                                      K, clip);
#undef B200W4A4_QLAUNCH
  return cudaGetLastError();
}

template <int PRE>
inline cudaError_t launch_quant_act_pre(const __half* x, void* q, float* scale, int M, int K,
                                        float clip, const PreArgs& pre, cudaStream_t stream) {
  const int nchunks = K / 8;
  if (nchunks > 256 * 8) return cudaErrorInvalidValue;  // rows must fit in registers (K <= 16384)
#define B200W4A4_QPLAUNCH(TPR, NCH)                                                             \
  do {                                                                                           \
    constexpr int ROWS = 256 / (TPR);                                                            \
    const unsigned grid = static_cast<unsigned>((static_cast<long long>(M) + ROWS - 1) / ROWS);  \
    quant_act_pre_rows_kernel<TPR, NCH, PRE><<<grid, 256, 0, stream>>>(x, q, scale, M, K, clip, pre); \
  } while (0)
  if (nchunks <= 32 * 6) B200W4A4_QPLAUNCH(32, 6);         // K = 1536
  else if (nchunks <= 32 * 8) B200W4A4_QPLAUNCH(32, 8);
  else if (nchunks <= 64 * 6) B200W4A4_QPLAUNCH(64, 6);    // K = 3072
  else if (nchunks <= 64 * 8) B200W4A4_QPLAUNCH(64, 8);
  else if (nchunks <= 128 * 5) B200W4A4_QPLAUNCH(128, 5);  // K = 5120
  else if (nchunks <= 128 * 8) B200W4A4_QPLAUNCH(128, 8);
  else B200W4A4_QPLAUNCH(256, 8);
#undef B200W4A4_QPLAUNCH
  return cudaGetLastError();
}

}  // namespace b200w4a4
