// Per-token work between the fused QKV projection and the attention kernel, in one pass:
//   RMSNorm over the whole row (all heads), rotary embedding, cast to the attention dtype.
//
// The reference runs these as separate PyTorch ops on [L, D] tensors
// (vdm_infer/models/wan_vdm/modules/attention.py: norm_q / norm_k :167-168 with the RMSNorm of
// :208-216, apply_rotary_emb :131-135, and the attention op's own dtype handling), i.e. about ten
// passes over q and k per block.  Here a row is read once, kept in registers, and written once.
//
// Rounding points are those of the reference ops so results agree to the last fp16 bit except
// where a reduction-order difference moves a value across a rounding boundary:
//   n   = fp16( float(x) * rsqrt(mean(float(x)^2) + eps) )
//   y   = fp16( n * w )                                   (fp16 multiply)
//   re  = fp16( y[2i]*cos - y[2i+1]*sin ),  im = fp16( y[2i]*sin + y[2i+1]*cos )   (fp32 arithmetic)
//   out = re/im as fp16, or rounded once more to bf16.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "quant_act.cuh"  // row_reduce

namespace b200w4a4 {

constexpr int kMaxPushDestinations = 8;

struct QkNormRopeArgs {
  const __half* x;            // [L, D], row pitch x_ld elements
  long long x_ld;
  const __half* weight;       // [D] or null: no normalisation
  const float* cos_sin;       // [L, head_dim/2, 2] (cos, sin) or null: no rotation
  float eps;
  int head_dim;
  void* out[8];               // destinations [>= out_row0 + L, D], row pitch out_ld elements, fp16 or bf16
  int n_out;                  // 1 = plain call; >1 = the same rows go to every destination (peer buffers)
  long long out_ld;
  long long out_row0;         // first destination row (this rank's offset inside a gathered buffer)
  // optional completion signal: after every store of the launch is visible system-wide,
  // flag[d][flag_index] = epoch for each destination d
  uint32_t* flag[8];
  int flag_index;
  uint32_t epoch;
  unsigned int* ticket;       // zero-initialised counter in this GPU's memory; left at zero again
  int L, D;
};


// TPR threads share a row; each holds up to NCH chunks of 8 consecutive values.
// PUSH: store to every destination and raise the completion flags; the plain instantiation
// writes out[0] only and carries none of that code.
template <int TPR, int NCH, bool OUT_BF16, bool PUSH>
__global__ void __launch_bounds__(256) qk_norm_rope_rows_kernel(const QkNormRopeArgs a) {
  constexpr int ROWS = 256 / TPR;
  __shared__ float red[8];
  const int sub = threadIdx.x / TPR;
  const int t = threadIdx.x % TPR;
  const long long row = static_cast<long long>(blockIdx.x) * ROWS + sub;
  const bool row_ok = row < a.L;
  const int nchunks = a.D >> 3;
  const __half* xr = a.x + (row_ok ? row : 0) * a.x_ld;

  uint4 raw[NCH];
#pragma unroll
  for (int i = 0; i < NCH; ++i) {
    const int c = t + i * TPR;
    raw[i] = make_uint4(0, 0, 0, 0);
    if (row_ok && c < nchunks) raw[i] = __ldcs(reinterpret_cast<const uint4*>(xr + 8 * c));
  }
  float r = 1.0f;
  if (a.weight != nullptr) {
    float ss = 0.0f;
#pragma unroll
    for (int i = 0; i < NCH; ++i) {
      const __half2* h = reinterpret_cast<const __half2*>(&raw[i]);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __half22float2(h[j]);
        ss = fmaf(f.x, f.x, ss);
        ss = fmaf(f.y, f.y, ss);
      }
    }
    ss = row_reduce<TPR, false>(ss, red, sub);
    r = rsqrtf(ss / static_cast<float>(a.D) + a.eps);
  }
  const float* cs_row = (a.cos_sin != nullptr) ? a.cos_sin + row * static_cast<long long>(a.head_dim) : nullptr;
  // 8 consecutive columns = 4 rotation pairs of one head (head_dim is a multiple of 8).  A thread's
  // chunks are TPR * 8 columns apart; when that is a whole number of heads they all sit at the same
  // offset inside their head, and the (cos, sin) pairs are fetched once instead of once per chunk.
  const bool cs_shared = (TPR * 8) % a.head_dim == 0;
  float4 cs0 = make_float4(1.f, 0.f, 1.f, 0.f), cs1 = cs0;
  if (cs_row != nullptr && cs_shared && row_ok && t < nchunks) {
    const int j0 = (8 * t) % a.head_dim;
    cs0 = __ldg(reinterpret_cast<const float4*>(cs_row + j0));
    cs1 = __ldg(reinterpret_cast<const float4*>(cs_row + j0) + 1);
  }
#pragma unroll
  for (int i = 0; i < NCH; ++i) {
    const int c = t + i * TPR;
    if (!row_ok || c >= nchunks) continue;
    const __half2* h = reinterpret_cast<const __half2*>(&raw[i]);
    __half2 y[4];
    if (a.weight != nullptr) {
      const uint4 wv = __ldg(reinterpret_cast<const uint4*>(a.weight + 8 * c));
      const __half2* w2 = reinterpret_cast<const __half2*>(&wv);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __half22float2(h[j]);
        const __half2 n = __floats2half2_rn(__fmul_rn(f.x, r), __fmul_rn(f.y, r));
        y[j] = __hmul2(n, w2[j]);
      }
    } else {
#pragma unroll
      for (int j = 0; j < 4; ++j) y[j] = h[j];
    }
    if (cs_row != nullptr) {
      if (!cs_shared) {
        const int j0 = (8 * c) % a.head_dim;
        cs0 = __ldg(reinterpret_cast<const float4*>(cs_row + j0));
        cs1 = __ldg(reinterpret_cast<const float4*>(cs_row + j0) + 1);
      }
      const float cc[4] = {cs0.x, cs0.z, cs1.x, cs1.z};
      const float sn[4] = {cs0.y, cs0.w, cs1.y, cs1.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __half22float2(y[j]);
        const float re = __fsub_rn(__fmul_rn(f.x, cc[j]), __fmul_rn(f.y, sn[j]));
        const float im = __fadd_rn(__fmul_rn(f.x, sn[j]), __fmul_rn(f.y, cc[j]));
        y[j] = __floats2half2_rn(re, im);
      }
    }
    uint4 o;
    uint32_t* ow = reinterpret_cast<uint32_t*>(&o);
    if constexpr (OUT_BF16) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __half22float2(y[j]);
        const __nv_bfloat162 b = __floats2bfloat162_rn(f.x, f.y);
        ow[j] = *reinterpret_cast<const uint32_t*>(&b);
      }
    } else {
#pragma unroll
      for (int j = 0; j < 4; ++j) ow[j] = *reinterpret_cast<const uint32_t*>(&y[j]);
    }
    // fp16 and bf16 are both two bytes wide: one element offset serves either type.
    const long long off = (a.out_row0 + row) * a.out_ld + 8 * c;
    if constexpr (PUSH) {
#pragma unroll
      for (int d = 0; d < kMaxPushDestinations; ++d)   // static indices: the pointers stay in the parameter bank
        if (d < a.n_out) *reinterpret_cast<uint4*>(static_cast<uint16_t*>(a.out[d]) + off) = o;
    } else {
      *reinterpret_cast<uint4*>(static_cast<uint16_t*>(a.out[0]) + off) = o;
    }
  }
  if (PUSH && a.ticket != nullptr) {
    // Publish: the barrier orders every thread's stores before thread 0, whose system-wide
    // fence then covers them all (fences are cumulative), and the ticket chain orders every
    // CTA's fence before the flag writes of the CTA that draws the last ticket.
    __syncthreads();
    if (threadIdx.x == 0) {
      __threadfence_system();
      const unsigned int t_last = gridDim.x - 1;
      if (atomicAdd(a.ticket, 1u) == t_last) {
        *a.ticket = 0u;
        __threadfence_system();
#pragma unroll
        for (int d = 0; d < kMaxPushDestinations; ++d) {
          if (d < a.n_out && a.flag[d] != nullptr)
            asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(a.flag[d] + a.flag_index), "r"(a.epoch) : "memory");
        }
      }
    }
  }
}

// Consumer side of the completion signal: one thread per flag waits, for a bounded time, until
// the flag has reached `epoch` (wrap-around safe).  A wait that runs out records
// DEV_TIMEOUT_PEER in the status word and returns; the context stays usable.
constexpr int DEV_TIMEOUT_PEER = 105;

__global__ void wait_flags_kernel(const uint32_t* flags, int n, uint32_t epoch, unsigned long long timeout_ns,
                                  int* status) {
  const int i = static_cast<int>(threadIdx.x);
  if (i >= n) return;
  unsigned long long t0 = 0;
  uint32_t spins = 0;
  while (true) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flags + i) : "memory");
    if (static_cast<int32_t>(v - epoch) >= 0) return;
    if ((++spins & 0xFF) == 0) {
      unsigned long long now;
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
      if (t0 == 0) {
        t0 = now;
      } else if (now - t0 > timeout_ns) {
        atomicCAS(status, 0, DEV_TIMEOUT_PEER);
        return;
      }
    }
  }
}

template <bool OUT_BF16, bool PUSH>
inline cudaError_t launch_qk_norm_rope(const QkNormRopeArgs& a, cudaStream_t stream) {
  const int nchunks = a.D / 8;
  if (nchunks > 256 * 8) return cudaErrorInvalidValue;  // a row must fit in registers (D <= 16384)
#define B200W4A4_GLUE_LAUNCH(TPR, NCH)                                                            \
  do {                                                                                             \
    constexpr int ROWS = 256 / (TPR);                                                              \
    const unsigned grid = static_cast<unsigned>((static_cast<long long>(a.L) + ROWS - 1) / ROWS);  \
    qk_norm_rope_rows_kernel<TPR, NCH, OUT_BF16, PUSH><<<grid, 256, 0, stream>>>(a);                     \
  } while (0)
  if (nchunks <= 32 * 4) B200W4A4_GLUE_LAUNCH(32, 4);
  else if (nchunks <= 32 * 8) B200W4A4_GLUE_LAUNCH(32, 8);
  else if (nchunks <= 64 * 8) B200W4A4_GLUE_LAUNCH(64, 8);
  else if (nchunks <= 128 * 5) B200W4A4_GLUE_LAUNCH(128, 5);  // D = 5120
  else if (nchunks <= 128 * 8) B200W4A4_GLUE_LAUNCH(128, 8);
  else B200W4A4_GLUE_LAUNCH(256, 8);
#undef B200W4A4_GLUE_LAUNCH
  return cudaGetLastError();
}

// Attention over the union of two disjoint key sets from the two partial results (what a rank
// computes when it attends to its own keys while the peers' keys are still arriving):
//   out = o1 * w1 + o2 * w2,  w_i = exp(l_i - logaddexp(l1, l2)),
// o_i bf16 [L, H*hd] (row pitch ld_i), l_i fp32 [H, L] log-sum-exp of the scaled scores, out bf16 [L, H*hd].
// One thread per 8 consecutive columns (one head never straddles a chunk: hd is a multiple of 8).
__global__ void __launch_bounds__(256)
attn_merge_kernel(const __nv_bfloat16* __restrict__ o1, const __nv_bfloat16* __restrict__ o2,
                  const float* __restrict__ lse1, const float* __restrict__ lse2,
                  __nv_bfloat16* __restrict__ out, int L, int H, int hd, long long ld1, long long ld2) {
  const int chunks = (H * hd) >> 3;
  const long long idx = static_cast<long long>(blockIdx.x) * 256 + threadIdx.x;
  if (idx >= static_cast<long long>(L) * chunks) return;
  const long long l = idx / chunks;
  const int c = static_cast<int>(idx % chunks);
  const int h = (8 * c) / hd;
  const float a = __ldg(lse1 + static_cast<long long>(h) * L + l);
  const float b = __ldg(lse2 + static_cast<long long>(h) * L + l);
  const float m = fmaxf(a, b);
  const float e1 = __expf(a - m), e2 = __expf(b - m);
  const float inv = 1.0f / (e1 + e2);
  const float w1 = e1 * inv, w2 = e2 * inv;
  const uint4 r1 = __ldcs(reinterpret_cast<const uint4*>(o1 + l * ld1 + 8 * c));
  const uint4 r2 = __ldcs(reinterpret_cast<const uint4*>(o2 + l * ld2 + 8 * c));
  const __nv_bfloat162* p1 = reinterpret_cast<const __nv_bfloat162*>(&r1);
  const __nv_bfloat162* p2 = reinterpret_cast<const __nv_bfloat162*>(&r2);
  uint4 o;
  __nv_bfloat162* po = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float2 f1 = __bfloat1622float2(p1[j]), f2 = __bfloat1622float2(p2[j]);
    po[j] = __floats2bfloat162_rn(fmaf(f1.x, w1, f2.x * w2), fmaf(f1.y, w1, f2.y * w2));
  }
  *reinterpret_cast<uint4*>(out + l * static_cast<long long>(H * hd) + 8 * c) = o;
}

// flag[d][index] = value on up to 8 flag arrays (this GPU's and peer-mapped ones), ordered after
// everything the stream ran before this kernel: "I am done reading" / "my part is complete".
struct SignalArgs {
  uint32_t* flag[kMaxPushDestinations];
  int n;
  int index;
  uint32_t value;
};

__global__ void signal_flags_kernel(const SignalArgs a) {
  const int d = static_cast<int>(threadIdx.x);
  if (d >= a.n) return;
  uint32_t* p = nullptr;
#pragma unroll
  for (int i = 0; i < kMaxPushDestinations; ++i)
    if (i == d) p = a.flag[i];
  if (p == nullptr) return;
  __threadfence_system();
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p + a.index), "r"(a.value) : "memory");
}

}  // namespace b200w4a4
