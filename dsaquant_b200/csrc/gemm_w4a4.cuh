// W4A4 GEMM for sm_100a:  out[m,n] = fp16( float(sum_k qa[m,k]*qw[n,k]) * (sa[m]*sw[n]) + bias[n] )
//
// Replaces linear_w4a4_kernel of the reference
// (vdm_infer/kernels/csrc/vdm_w4a4_kernel.cu:627-686, mma.sync m16n8k64 s4 fed
// from registers) with a persistent, warp-specialised tcgen05 kernel:
//
//   warp 0       TMA producer: activation codes (int8 container, K-major, 128B swizzle)
//   warp 1       owns TMEM; one lane issues tcgen05.mma kind::i8 (K=32 slices)
//   warp 2       TMA producer: packed int4 weight tiles (two codes per byte)
//   warps 3-6    unpack the int4 weight tile into the int8 K-major/128B-swizzle
//                tile the tensor core reads (tcgen05 has no s4 kind)
//   warps 7-14   epilogue: tcgen05.ld the int32 accumulator, dequantise with the
//                per-token x per-channel scales, add bias, fp16, TMA store
//
// Weight nibble convention (produced by the load-time repack, see
// weight_pack.cuh): inside each 128-wide K block, byte (16*c + i) of a row
// holds code[k0+32c+i] in its HIGH nibble and code[k0+32c+16+i] in its LOW
// nibble.  `p & 0xF0F0F0F0` and `(p << 4) & 0xF0F0F0F0` are then two runs of
// 16 consecutive-k int8 values equal to 16*code: no sign extension is needed.
// The int32 accumulator comes out multiplied by 16 and the epilogue undoes it
// with an exact arithmetic shift, so accumulators stay bit-exact.
//
// CG == 1: one CTA computes a 128 x 256 tile.  CG == 2: a CTA pair computes a
// 256 x 256 tile with cta_group::2 MMAs; each CTA stages its own 128 rows of A
// and unpacks its own 128 weight rows, halving per-SM shared-memory traffic.
#pragma once
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "ptx.cuh"

namespace b200w4a4 {

// Device status codes written by a kernel whose bounded wait ran out.
enum : int {
  DEV_OK = 0,
  DEV_TIMEOUT_PRODUCER = 101,
  DEV_TIMEOUT_UNPACK = 102,
  DEV_TIMEOUT_MMA = 103,
  DEV_TIMEOUT_EPILOGUE = 104,
};

// W8: the weight operand is already int8 in global memory (every byte 16 * code, written by the
// load-time expansion) and TMA stages it straight into the tile the tensor core reads: no packed
// ring, no unpack warps' work, one more main-ring stage -- at twice the weight bytes in HBM and L2.
template <int CG, bool W8 = false>
struct GemmCfg {
  static constexpr int BM = 128;                 // rows of A per CTA
  static constexpr int BN = 256;                 // output columns per tile
  static constexpr int BK = 128;                 // k per pipeline stage (one 128B swizzle row)
  static constexpr int B_ROWS = BN / CG;         // weight rows staged + unpacked per CTA
  static constexpr int A_BYTES = BM * BK;        // int8
  static constexpr int BP_BYTES = B_ROWS * BK / 2;
  static constexpr int BU_BYTES = B_ROWS * BK;
  // Main ring: one stage = an A tile (TMA) + an unpacked weight tile; released by one MMA commit.
  // Packed weight tiles live in a second, shallower ring that is released as soon as they have
  // been unpacked.
  static constexpr int S = (CG == 1) ? (W8 ? 4 : 3) : (W8 ? 6 : 5);
  static constexpr int SB = W8 ? 0 : ((CG == 1) ? 3 : 4);
  static constexpr int STAGE_BYTES = A_BYTES + BU_BYTES;
  static constexpr int EPI_BUF = 32 * 128;       // 32 rows x 64 fp16: one TMA store box
  static constexpr int EPI_WARPS = 8;             // two warps per TMEM lane quadrant, half the columns each
  // Staging buffers per epilogue warp.  Two (a warp fills one while the TMA store of the other
  // still reads shared memory) fit only by giving up the fifth main-ring stage; measured, that
  // trade changed nothing at K = 1536 and cost 3-6 % at K >= 8960, so one buffer it is.
  static constexpr int EPI_STAGES = 1;
  static constexpr int EPI_BYTES = EPI_WARPS * EPI_STAGES * EPI_BUF;
  static constexpr int OFF_MAIN = 0;
  static constexpr int OFF_BP = OFF_MAIN + S * STAGE_BYTES;
  static constexpr int OFF_EPI = OFF_BP + SB * BP_BYTES;
  static constexpr int OFF_BAR = OFF_EPI + EPI_BYTES;
  static constexpr int NUM_BARS = 2 * S + 2 * SB + 4 + 1;
  static constexpr int SMEM_BYTES = OFF_BAR + 8 * NUM_BARS + 16;
  static constexpr int SMEM_ALLOC = SMEM_BYTES + 1024;  // slack to align the base to 1024 B
  static constexpr int WARP_A_PRODUCER = 0, WARP_MMA = 1, WARP_B_PRODUCER = 2;
  static constexpr int WARP_UNPACK0 = 3, UNPACK_WARPS = 4, WARP_EPI0 = WARP_UNPACK0 + UNPACK_WARPS;
  static constexpr int UNPACK_THREADS = 32 * UNPACK_WARPS;
  static constexpr int THREADS = 32 * (WARP_EPI0 + EPI_WARPS);
  static constexpr int TMEM_COLS = 512;          // two 128 x 256 int32 accumulators
  static constexpr int GROUP_M = 8;              // tile rasterisation: walk 8 row-tiles per column-tile
  static_assert(BP_BYTES % 1024 == 0 && BU_BYTES % 1024 == 0 && A_BYTES % 1024 == 0, "alignment");
  static_assert((B_ROWS * 4) % UNPACK_THREADS == 0, "unpack work split");
  static_assert(((BN / 32) / (EPI_WARPS / 4)) % 2 == 0, "the epilogue loads TMEM two chunks at a time");
  static_assert(SMEM_ALLOC <= 232448, "shared memory budget");
};

// 64-bit shared-memory matrix descriptor, K-major, 128-byte swizzle, 8-row
// groups 1024 B apart (bit layout: start>>4 [0,14), LBO>>4 [16,30),
// SBO>>4 [32,46), version=1 [46,48), layout type 2 = SWIZZLE_128B [61,64)).
__device__ __forceinline__ uint64_t make_kmajor_sw128_desc(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFF) >> 4);
  d |= static_cast<uint64_t>(1) << 16;
  d |= static_cast<uint64_t>(1024 >> 4) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(2) << 61;
  return d;
}

// 32-bit instruction descriptor for kind::i8: D=s32 (2 @ bit 4), A=s8 (1 @ bit 7),
// B=s8 (1 @ bit 10), both K-major, N>>3 @ bit 17, M>>4 @ bit 24.
__host__ __device__ constexpr uint32_t make_i8_idesc(int m, int n) {
  return (2u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(n >> 3) << 17) |
         (static_cast<uint32_t>(m >> 4) << 24);
}

struct GemmParams {
  const float* act_scale;   // [M] fp32
  const __half* w_scale;    // [N] fp16
  const __half* bias;       // [N] fp16 or null
  int32_t* acc_dump;        // [M,N] int32 or null (tests)
  int M, N, K;
  int m_tiles, n_tiles;     // in units of (CG*128) rows and 256 columns
  int* status;              // device status word: first time-out code of any launch (report only)
  unsigned* abort_word;     // holds the id of the launch that last timed out
  unsigned launch_id;       // id of this launch (never 0): only its own time-out cancels it
  // epilogue extras (see the EPI_* variants)
  const __half* residual;   // [M,N] fp16, may alias the output
  const float* gate;        // [N] (or [M,N] with gate_row_stride = N)
  long long gate_row_stride;
  int seg_cols;             // EPI_SPLIT: width of one output segment (N / segments, a multiple of 64)
};

// Tensor maps of the output: one [M,N] matrix, or (EPI_SPLIT) up to three [M,seg_cols]
// matrices with their own base pointers and row strides.
struct OutMaps {
  CUtensorMap seg[3];
};

// Work fused behind the dequantisation (what the caller would otherwise run as separate
// elementwise kernels over the [M,N] output).  y16 = fp16(acc * sa * sw + bias) in every case.
enum : int {
  EPI_NONE = 0,           // out = y16
  EPI_GELU_TANH = 1,      // out = fp16(gelu_tanh(y16))                        FFN up projection
  EPI_GATE_RESIDUAL = 2,  // out = fp16(float(residual) + float(y16) * gate)   attention / FFN output + skip
  EPI_SPLIT = 3,          // out_s[m, n - s*seg_cols] = y16 with s = n / seg_cols   fused QKV / KV projections
};

namespace detail {

constexpr uint64_t kWaitLimitNs = 1000ull * 1000ull * 1000ull;  // 1 s per wait

// What a bounded wait needs to give up cleanly.  The status word is only a report (it keeps the
// first code until the host reads it, and other kernels write to it too), so it never cancels a
// launch; the abort word does, and only for the launch whose id it holds.
struct WaitCtx {
  volatile int* abort_flag;  // CTA-local, shared memory
  int* status;
  unsigned* abort_word;
  unsigned launch_id;
};

// Bounded wait on an mbarrier phase.  On time-out records `code` once, publishes this launch's
// id in the abort word, raises the CTA-local abort flag and returns false; every other role sees
// the flag (or, in another CTA, the abort word) in its own wait and drains too.
__device__ __forceinline__ bool wait_bar(uint32_t bar, uint32_t parity, const WaitCtx& w, int code) {
  if (ptx::mbar_probe(bar, parity)) return true;
  uint32_t spins = 0;
  uint64_t t0 = 0;
  while (true) {
    if (ptx::mbar_test(bar, parity)) return true;
    if ((++spins & 0x3FF) == 0) {
      if (*w.abort_flag) return false;
      if (*reinterpret_cast<volatile unsigned*>(w.abort_word) == w.launch_id) {
        *w.abort_flag = 1;
        return false;
      }
      uint64_t now = ptx::globaltimer_ns();
      if (t0 == 0) {
        t0 = now;
      } else if (now - t0 > kWaitLimitNs) {
        atomicCAS(w.status, 0, code);
        atomicExch(w.abort_word, w.launch_id);
        *w.abort_flag = 1;
        return false;
      }
    }
  }
}

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

__device__ __forceinline__ uint4 lds128(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "r"(addr));
  return v;
}
__device__ __forceinline__ void sts128(uint32_t addr, uint4 v) {
  asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z),
               "r"(v.w)
               : "memory");
}

}  // namespace detail

// Tile index -> (row tile, column tile).  Consecutive indices walk GROUP_M row tiles of one
// column tile before moving to the next column tile, so the CTAs that run at the same time share
// both their activation rows and their weight rows through L2 instead of all fetching one of them.
template <int CG>
__device__ __forceinline__ void tile_coords(int tile, int m_tiles, int n_tiles, int& mt, int& nt) {
  constexpr int G = GemmCfg<CG>::GROUP_M;
  const int per_group = G * n_tiles;
  const int group = tile / per_group;
  const int first_m = group * G;
  const int rows = (m_tiles - first_m < G) ? (m_tiles - first_m) : G;
  const int in_group = tile - group * per_group;
  mt = first_m + in_group % rows;
  nt = in_group / rows;
}

// Ring cursor: slot index and phase parity, advanced without division.
template <int DEPTH>
struct RingPos {
  uint32_t slot = 0, phase = 0;
  __device__ __forceinline__ void advance() {
    if (++slot == DEPTH) {
      slot = 0;
      phase ^= 1;
    }
  }
};

__device__ __forceinline__ float epi_gelu_tanh(float x) {
  const float kBeta = 0.7978845608028654f;  // sqrt(2/pi)
  const float kKappa = 0.044715f;
  const float x3 = x * x * x;
  const float inner = kBeta * (x + kKappa * x3);
  return 0.5f * x * (1.0f + tanhf(inner));
}

template <int CG, int EPI = EPI_NONE, bool W8 = false>
__global__ void __launch_bounds__(GemmCfg<CG, W8>::THREADS, 1)
gemm_w4a4_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_w,
                 const __grid_constant__ OutMaps tm_out, const GemmParams p) {
  using C = GemmCfg<CG, W8>;
  extern __shared__ uint8_t smem_raw[];
  // 128B-swizzled tiles want a 1024 B aligned base.
  const uint32_t smem_base = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - ptx::smem_u32(smem_raw));

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t cta_rank = (CG == 2) ? detail::cluster_ctarank() : 0u;
  const bool leader = (cta_rank == 0);

  // ---- barrier map ---------------------------------------------------------
  // full[s]      A bytes landed (TMA transaction count) AND every unpack warp of the group has
  //              written its part of the int8 weight tile: the one barrier the MMA waits on.
  // consumed[s]  the MMAs that read stage s have completed (tcgen05.commit): frees A and Bu.
  const uint32_t bar0 = smem_base + C::OFF_BAR;
  auto bar_full = [&](uint32_t s) { return bar0 + 8u * s; };
  auto bar_consumed = [&](uint32_t s) { return bar0 + 8u * (C::S + s); };
  auto bar_bp_full = [&](uint32_t s) { return bar0 + 8u * (2 * C::S + s); };
  auto bar_bp_free = [&](uint32_t s) { return bar0 + 8u * (2 * C::S + C::SB + s); };
  auto bar_acc_full = [&](uint32_t b) { return bar0 + 8u * (2 * C::S + 2 * C::SB + b); };
  auto bar_acc_free = [&](uint32_t b) { return bar0 + 8u * (2 * C::S + 2 * C::SB + 2 + b); };
  volatile int* abort_flag =
      reinterpret_cast<volatile int*>(smem_gen + C::OFF_BAR + 8 * (C::NUM_BARS - 1));
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(smem_gen + C::OFF_BAR + 8 * C::NUM_BARS);
  const detail::WaitCtx wctx{abort_flag, p.status, p.abort_word, p.launch_id};

  if (threadIdx.x == 0) {
    for (int s = 0; s < C::S; ++s) {
      ptx::mbar_init(bar_full(s), W8 ? 1 : C::UNPACK_WARPS * CG + 1);  // unpack warps + the A producer
      ptx::mbar_init(bar_consumed(s), 1);                     // one MMA commit
    }
    for (int s = 0; s < C::SB; ++s) {
      ptx::mbar_init(bar_bp_full(s), 1);
      ptx::mbar_init(bar_bp_free(s), C::UNPACK_WARPS);
    }
    for (int b = 0; b < 2; ++b) {
      ptx::mbar_init(bar_acc_full(b), 1);
      ptx::mbar_init(bar_acc_free(b), C::EPI_WARPS * CG);  // epilogue warps of every CTA in the group
    }
    *abort_flag = 0;
    ptx::fence_mbar_init();
  }
  if (warp == C::WARP_A_PRODUCER && lane == 0) {
    ptx::prefetch_tensormap(&tm_a);
    ptx::prefetch_tensormap(&tm_w);
    ptx::prefetch_tensormap(&tm_out.seg[0]);
  }
  if (warp == C::WARP_MMA) {
    ptx::tmem_alloc<CG>(ptx::smem_u32(tmem_holder), C::TMEM_COLS);
    ptx::tmem_relinquish<CG>();
  }
  ptx::tc_fence_before_sync();
  __syncthreads();
  if constexpr (CG == 2) detail::cluster_sync_all();
  ptx::tc_fence_after_sync();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_holder);

  // ---- persistent tile loop bookkeeping -----------------------------------
  const int num_tiles = p.m_tiles * p.n_tiles;
  const int first_tile = static_cast<int>(blockIdx.x) / CG;
  const int tile_step = static_cast<int>(gridDim.x) / CG;
  const int kblocks = (p.K + C::BK - 1) / C::BK;

  if (warp == C::WARP_A_PRODUCER) {
    // ===================== TMA producer: activation codes =====================
    if (lane == 0) {
      RingPos<C::S> pos;
      bool alive = true;
      // Both CTAs of a pair feed the leader's MMA: byte counts go to the leader's barrier.
      uint32_t full_remote[C::S];
#pragma unroll
      for (int s = 0; s < C::S; ++s) full_remote[s] = (CG == 2) ? ptx::mapa(bar_full(s), 0) : 0u;
      for (int tile = first_tile; tile < num_tiles && alive; tile += tile_step) {
        int mt, nt;
        tile_coords<CG>(tile, p.m_tiles, p.n_tiles, mt, nt);
        const int m0 = mt * (C::BM * CG) + static_cast<int>(cta_rank) * C::BM;
        for (int kb = 0; kb < kblocks; ++kb) {
          if (!detail::wait_bar(bar_consumed(pos.slot), pos.phase ^ 1, wctx,
                                DEV_TIMEOUT_PRODUCER)) {
            alive = false;
            break;
          }
          const uint32_t dst = smem_base + C::OFF_MAIN + pos.slot * C::STAGE_BYTES;
          if constexpr (W8) {
            const int n0w = nt * C::BN + static_cast<int>(cta_rank) * C::B_ROWS;
            if constexpr (CG == 1) {
              ptx::mbar_arrive_expect_tx(bar_full(pos.slot), C::A_BYTES + C::BU_BYTES);
              ptx::tma_load_2d(dst, &tm_a, bar_full(pos.slot), kb * C::BK, m0);
              ptx::tma_load_2d(dst + C::A_BYTES, &tm_w, bar_full(pos.slot), kb * C::BK, n0w);
            } else {
              if (leader) ptx::mbar_arrive_expect_tx(bar_full(pos.slot), 2 * (C::A_BYTES + C::BU_BYTES));
              uint32_t remote = full_remote[0];
  #pragma unroll
              for (int s = 1; s < C::S; ++s) remote = (pos.slot == s) ? full_remote[s] : remote;
              ptx::tma_load_2d_pair(dst, &tm_a, remote, kb * C::BK, m0);
              ptx::tma_load_2d_pair(dst + C::A_BYTES, &tm_w, remote, kb * C::BK, n0w);
            }
          } else {
            if constexpr (CG == 1) {
              ptx::mbar_arrive_expect_tx(bar_full(pos.slot), C::A_BYTES);
              ptx::tma_load_2d(dst, &tm_a, bar_full(pos.slot), kb * C::BK, m0);
            } else {
              if (leader) ptx::mbar_arrive_expect_tx(bar_full(pos.slot), 2 * C::A_BYTES);
              uint32_t remote = full_remote[0];
  #pragma unroll
              for (int s = 1; s < C::S; ++s) remote = (pos.slot == s) ? full_remote[s] : remote;
              ptx::tma_load_2d_pair(dst, &tm_a, remote, kb * C::BK, m0);
            }
          }
          pos.advance();
        }
      }
      if (!alive) {
        // Drain: give loads already issued a bounded time to land before smem goes away.
        const uint64_t t0 = ptx::globaltimer_ns();
        while (ptx::globaltimer_ns() - t0 < 2000000ull) {
        }
      }
    }
  } else if (warp == C::WARP_B_PRODUCER) {
    // ===================== TMA producer: packed int4 weights =====================
    if (lane == 0 && !W8) {
      RingPos<C::SB> pos;
      bool alive = true;
      // Weights are re-read by every row tile: ask L2 to keep them while outputs stream through.
      const uint64_t keep = ptx::l2_policy_evict_last();
      for (int tile = first_tile; tile < num_tiles && alive; tile += tile_step) {
        int mt, nt;
        tile_coords<CG>(tile, p.m_tiles, p.n_tiles, mt, nt);
        const int n0 = nt * C::BN + static_cast<int>(cta_rank) * C::B_ROWS;
        for (int kb = 0; kb < kblocks; ++kb) {
          if (!detail::wait_bar(bar_bp_free(pos.slot), pos.phase ^ 1, wctx,
                                DEV_TIMEOUT_PRODUCER)) {
            alive = false;
            break;
          }
          ptx::mbar_arrive_expect_tx(bar_bp_full(pos.slot), C::BP_BYTES);
          ptx::tma_load_2d_hint(smem_base + C::OFF_BP + pos.slot * C::BP_BYTES, &tm_w,
                                bar_bp_full(pos.slot), kb * (C::BK / 2), n0, keep);
          pos.advance();
        }
      }
      if (!alive) {
        const uint64_t t0 = ptx::globaltimer_ns();
        while (ptx::globaltimer_ns() - t0 < 2000000ull) {
        }
      }
    }
  } else if (warp == C::WARP_MMA) {
    // ===================== MMA issuer =====================
    // One thread issues every MMA of the group and its loop is the critical path of the kernel
    // (measured: every instruction added here lengthens each stage by its latency).  It is
    // therefore unrolled over the ring slots so that barrier addresses and descriptor words are
    // loop-invariant registers, and a stage costs one barrier probe, four MMAs and one commit.
    if (lane == 0 && (CG == 1 || leader)) {
      constexpr uint32_t idesc = make_i8_idesc(C::BM * CG, C::BN);
      const uint64_t adesc0 = make_kmajor_sw128_desc(smem_base + C::OFF_MAIN);
      const uint64_t bdesc0 = make_kmajor_sw128_desc(smem_base + C::OFF_MAIN + C::A_BYTES);
      const uint32_t a_hi = static_cast<uint32_t>(adesc0 >> 32), b_hi = static_cast<uint32_t>(bdesc0 >> 32);
      const uint32_t a_lo0 = static_cast<uint32_t>(adesc0), b_lo0 = static_cast<uint32_t>(bdesc0);
      auto commit_to = [&](uint32_t bar) {
        if constexpr (CG == 1)
          ptx::mma_commit(bar);
        else
          ptx::mma_commit_pair(bar, 0x3);
      };
      int tile = first_tile;
      bool running = tile < num_tiles;
      uint32_t local_tile = 0, phase = 0;
      int kb = 0;
      uint32_t tmem_d = tmem_base;
      while (running) {
#pragma unroll
        for (int s = 0; s < C::S; ++s) {
          if (!running) break;
          if (kb == 0) {
            const uint32_t ab = local_tile & 1;
            if (!detail::wait_bar(bar_acc_free(ab), ((local_tile >> 1) & 1) ^ 1, wctx, DEV_TIMEOUT_MMA)) {
              running = false;
              break;
            }
            tmem_d = tmem_base + ab * C::BN;
            ptx::tc_fence_after_sync();  // orders the epilogue's TMEM reads before this tile's MMAs
          }
          if (!detail::wait_bar(bar_full(s), phase, wctx, DEV_TIMEOUT_MMA)) {
            running = false;
            break;
          }
          // +32 bytes along K inside the 128B swizzle row = +2 in the (addr >> 4) field.
          const uint32_t a_lo = a_lo0 + s * (C::STAGE_BYTES >> 4), b_lo = b_lo0 + s * (C::STAGE_BYTES >> 4);
          ptx::mma_i8_ss_lohi<CG>(tmem_d, a_lo, a_hi, b_lo, b_hi, idesc, kb > 0 ? 1u : 0u);
          ptx::mma_i8_ss_lohi<CG>(tmem_d, a_lo + 2u, a_hi, b_lo + 2u, b_hi, idesc, 1u);
          ptx::mma_i8_ss_lohi<CG>(tmem_d, a_lo + 4u, a_hi, b_lo + 4u, b_hi, idesc, 1u);
          ptx::mma_i8_ss_lohi<CG>(tmem_d, a_lo + 6u, a_hi, b_lo + 6u, b_hi, idesc, 1u);
          commit_to(bar_consumed(s));
          if (++kb == kblocks) {
            commit_to(bar_acc_full(local_tile & 1));
            kb = 0;
            ++local_tile;
            tile += tile_step;
            running = tile < num_tiles;
          }
        }
        phase ^= 1;
      }
    }
  } else if (warp < C::WARP_EPI0) {
    // ===================== int4 -> int8 weight unpack =====================
    const int tid_u = static_cast<int>(threadIdx.x) - 32 * C::WARP_UNPACK0;
    const uint32_t row_x = static_cast<uint32_t>((tid_u >> 2) & 7);
    const uint32_t c2 = static_cast<uint32_t>(tid_u & 3) * 2;
    const uint32_t hi_off = ((c2 ^ row_x) << 4);
    const uint32_t lo_off = (((c2 + 1) ^ row_x) << 4);
    RingPos<C::S> pos;
    RingPos<C::SB> bpos;
    bool alive = !W8;
    for (int tile = first_tile; tile < num_tiles && alive; tile += tile_step) {
      for (int kb = 0; kb < kblocks; ++kb) {
        if (!detail::wait_bar(bar_bp_full(bpos.slot), bpos.phase, wctx, DEV_TIMEOUT_UNPACK) ||
            !detail::wait_bar(bar_consumed(pos.slot), pos.phase ^ 1, wctx, DEV_TIMEOUT_UNPACK)) {
          alive = false;
          break;
        }
        const uint32_t bp = smem_base + C::OFF_BP + bpos.slot * C::BP_BYTES;
        const uint32_t bu = smem_base + C::OFF_MAIN + pos.slot * C::STAGE_BYTES + C::A_BYTES;
        constexpr int ITERS = C::B_ROWS * 4 / C::UNPACK_THREADS;
        uint4 pk[ITERS];
#pragma unroll
        for (int j = 0; j < ITERS; ++j)
          pk[j] = detail::lds128(bp + 16u * static_cast<uint32_t>(tid_u + C::UNPACK_THREADS * j));
#pragma unroll
        for (int j = 0; j < ITERS; ++j) {
          const int q = tid_u + C::UNPACK_THREADS * j;  // 16-byte packed chunk index in the tile
          uint4 hi, lo;
          hi.x = pk[j].x & 0xF0F0F0F0u; lo.x = (pk[j].x << 4) & 0xF0F0F0F0u;
          hi.y = pk[j].y & 0xF0F0F0F0u; lo.y = (pk[j].y << 4) & 0xF0F0F0F0u;
          hi.z = pk[j].z & 0xF0F0F0F0u; lo.z = (pk[j].z << 4) & 0xF0F0F0F0u;
          hi.w = pk[j].w & 0xF0F0F0F0u; lo.w = (pk[j].w << 4) & 0xF0F0F0F0u;
          const uint32_t row_addr = bu + 128u * static_cast<uint32_t>(q >> 2);
          detail::sts128(row_addr + hi_off, hi);
          detail::sts128(row_addr + lo_off, lo);
        }
        // Generic-proxy writes must be visible to the tensor core's async-proxy reads.
        ptx::fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          ptx::mbar_arrive(bar_bp_free(bpos.slot));
          if constexpr (CG == 1)
            ptx::mbar_arrive(bar_full(pos.slot));
          else
            ptx::mbar_arrive_cluster(bar_full(pos.slot), 0);
        }
        pos.advance();
        bpos.advance();
      }
    }
  } else {
    // ===================== epilogue =====================
    const int quad = warp & 3;  // TMEM lane quadrant this warp may read
    const uint32_t stage_buf0 = smem_base + C::OFF_EPI + (warp - C::WARP_EPI0) * (C::EPI_STAGES * C::EPI_BUF);
    const uint32_t row_sw = static_cast<uint32_t>(lane & 7);
    uint32_t local_tile = 0;
    bool alive = true;
    // The output is written once and not read by this kernel: evict it first, so that it does
    // not push the weights (re-read by every row tile) out of L2.
    const uint64_t stream_out = ptx::l2_policy_evict_first();
    for (int tile = first_tile; tile < num_tiles && alive; tile += tile_step, ++local_tile) {
      int mt, nt;
      tile_coords<CG>(tile, p.m_tiles, p.n_tiles, mt, nt);
      const int m0 = mt * (C::BM * CG) + static_cast<int>(cta_rank) * C::BM + quad * 32;
      const int n0 = nt * C::BN;
      const uint32_t ab = local_tile & 1;
      const uint32_t aph = (local_tile >> 1) & 1;
      if (!detail::wait_bar(bar_acc_full(ab), aph, wctx, DEV_TIMEOUT_EPILOGUE)) {
        alive = false;
        break;
      }
      ptx::tc_fence_after_sync();
      const int row = m0 + lane;
      const float sa = (row < p.M) ? __ldg(p.act_scale + row) : 0.0f;
      const bool small_k = p.K < 16384;                   // 16 * 64 * K < 2^24
      const float sa_eff = small_k ? sa * 0.0625f : sa;   // exact: power-of-two scaling
      const int unshift = small_k ? 0 : 4;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + ab * C::BN;
      // Warps e and e+4 share a lane quadrant and split the tile's columns.
      constexpr int CHUNKS = (C::BN / 32) / (C::EPI_WARPS / 4);
      const int c_first = ((warp - C::WARP_EPI0) >> 2) * CHUNKS;
      // A 64-column store box is filled by two consecutive 32-column chunks; boxes alternate
      // between the warp's staging buffers.
      auto process = [&](uint32_t (&acc)[32], const int c) {
        const uint32_t stage_buf = stage_buf0 + (C::EPI_STAGES == 2 ? (((c - c_first) >> 1) & 1) * C::EPI_BUF : 0);
        const uint32_t stage = stage_buf + 128u * lane;
        const int col0 = n0 + 32 * c;
        const bool cols_valid = col0 < p.N;  // N is a multiple of 128: a 32-chunk is all in or all out
        uint4 packed4[4];
        if (cols_valid) {
          if (p.acc_dump != nullptr && row < p.M) {
            int4* dst = reinterpret_cast<int4*>(p.acc_dump + static_cast<size_t>(row) * p.N + col0);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              dst[i] = make_int4(static_cast<int>(acc[4 * i]) >> 4, static_cast<int>(acc[4 * i + 1]) >> 4,
                                 static_cast<int>(acc[4 * i + 2]) >> 4,
                                 static_cast<int>(acc[4 * i + 3]) >> 4);
            }
          }
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            const uint4 wsv = __ldg(reinterpret_cast<const uint4*>(p.w_scale + col0 + 8 * g));
            uint4 bv = make_uint4(0, 0, 0, 0);
            if (p.bias != nullptr) bv = __ldg(reinterpret_cast<const uint4*>(p.bias + col0 + 8 * g));
            const __half2* ws2 = reinterpret_cast<const __half2*>(&wsv);
            const __half2* b2 = reinterpret_cast<const __half2*>(&bv);
            uint4 resv = make_uint4(0, 0, 0, 0);
            float gt[8] = {0, 0, 0, 0, 0, 0, 0, 0};
            if constexpr (EPI == EPI_GATE_RESIDUAL) {
              if (row < p.M) {
                resv = *reinterpret_cast<const uint4*>(p.residual + static_cast<size_t>(row) * p.N + col0 + 8 * g);
                const float* gp = p.gate + row * p.gate_row_stride + col0 + 8 * g;
                const float4 g0 = __ldg(reinterpret_cast<const float4*>(gp));
                const float4 g1 = __ldg(reinterpret_cast<const float4*>(gp) + 1);
                gt[0] = g0.x; gt[1] = g0.y; gt[2] = g0.z; gt[3] = g0.w;
                gt[4] = g1.x; gt[5] = g1.y; gt[6] = g1.z; gt[7] = g1.w;
              }
            }
            const __half2* r2 = reinterpret_cast<const __half2*>(&resv);
            uint32_t packed[4];
#pragma unroll
            for (int h = 0; h < 4; ++h) {
              const float2 wsf = __half22float2(ws2[h]);
              const float2 bf = __half22float2(b2[h]);
              // Every weight byte was 16 * code, so the accumulator is 16 * acc.  With
              // |16 * acc| < 2^24 the conversion to fp32 is exact and the factor moves into the
              // scale product as an exact power of two: fl((16 acc) * fl((sa / 16) * sw)) == fl(acc * fl(sa * sw)).
              // Longer reductions undo it with an exact arithmetic shift first.
              const int i0 = static_cast<int>(acc[8 * g + 2 * h]), i1 = static_cast<int>(acc[8 * g + 2 * h + 1]);
              const float a0 = static_cast<float>(i0 >> unshift);
              const float a1 = static_cast<float>(i1 >> unshift);
              float v0 = __fmul_rn(a0, __fmul_rn(sa_eff, wsf.x));
              float v1 = __fmul_rn(a1, __fmul_rn(sa_eff, wsf.y));
              if (p.bias != nullptr) {
                v0 = __fadd_rn(v0, bf.x);
                v1 = __fadd_rn(v1, bf.y);
              }
              __half2 o = __floats2half2_rn(v0, v1);
              if constexpr (EPI == EPI_GELU_TANH) {
                const float2 y = __half22float2(o);
                o = __floats2half2_rn(epi_gelu_tanh(y.x), epi_gelu_tanh(y.y));
              } else if constexpr (EPI == EPI_GATE_RESIDUAL) {
                const float2 y = __half22float2(o);
                const float2 rf = __half22float2(r2[h]);
                o = __floats2half2_rn(__fadd_rn(rf.x, __fmul_rn(y.x, gt[2 * h])),
                                      __fadd_rn(rf.y, __fmul_rn(y.y, gt[2 * h + 1])));
              }
              packed[h] = *reinterpret_cast<const uint32_t*>(&o);
            }
            packed4[g] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
          }
        }
        if ((c & 1) == 0) {
          // The store that last used this staging buffer must have finished reading it (with two
          // buffers that is the store before the previous one); waiting here, after the
          // arithmetic, lets that read overlap this chunk's dequantisation.
          if (lane == 0) ptx::tma_store_wait_read<C::EPI_STAGES - 1>();
          __syncwarp();
        }
        if (cols_valid) {
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            const uint32_t chunk = static_cast<uint32_t>((c & 1) * 4 + g);
            detail::sts128(stage + ((chunk ^ row_sw) << 4), packed4[g]);
          }
        }
        if ((c & 1) == 1) {
          ptx::fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            const int c_store = col0 - 32;
            if (c_store < p.N && m0 < p.M) {
              if constexpr (EPI == EPI_SPLIT) {
                // seg_cols is a multiple of the 64-column store box, so a box lies in one segment.
                const int sgm = c_store / p.seg_cols;
                ptx::tma_store_2d_hint(&tm_out.seg[sgm], stage_buf, c_store - sgm * p.seg_cols, m0, stream_out);
              } else {
                ptx::tma_store_2d_hint(&tm_out.seg[0], stage_buf, c_store, m0, stream_out);
              }
            }
            ptx::tma_store_commit();
          }
        }
      };
      // TMEM reads run one chunk ahead of the arithmetic: while chunk c is dequantised and staged,
      // the load of chunk c + 1 is in flight.
      auto release_accumulator = [&]() {
        // Accumulator fully read: hand the TMEM buffer back to the MMA warp.
        ptx::tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) {
          if constexpr (CG == 1)
            ptx::mbar_arrive(bar_acc_free(ab));
          else
            ptx::mbar_arrive_cluster(bar_acc_free(ab), 0);
        }
      };
      uint32_t acc_a[32], acc_b[32];
      ptx::tmem_ld_32x32(taddr + 32u * c_first, acc_a);
#pragma unroll 1
      for (int c = c_first; c < c_first + CHUNKS; c += 2) {
        ptx::tmem_ld_wait_for(acc_a);
        ptx::tmem_ld_32x32(taddr + 32u * (c + 1), acc_b);
        process(acc_a, c);
        ptx::tmem_ld_wait_for(acc_b);
        if (c + 2 < c_first + CHUNKS)
          ptx::tmem_ld_32x32(taddr + 32u * (c + 2), acc_a);
        else
          release_accumulator();
        process(acc_b, c + 1);
      }
    }
    if (lane == 0) ptx::tma_store_wait_all<0>();
  }

  // ---- teardown --------------------------------------------------------------
  ptx::tc_fence_before_sync();
  __syncthreads();
  if constexpr (CG == 2) detail::cluster_sync_all();
  if (warp == C::WARP_MMA) {
    __syncwarp();
    ptx::tc_fence_after_sync();
    ptx::tmem_dealloc<CG>(tmem_base, C::TMEM_COLS);
  }
}

}  // namespace b200w4a4
