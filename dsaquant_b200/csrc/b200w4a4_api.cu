// C-ABI entry points of libb200w4a4.so (declared in include/b200w4a4.h).
// Host side only: argument checks, TMA descriptor encoding, kernel launches.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>

#include <string.h>

#include <atomic>
#include <mutex>
#include <unordered_map>

#include "../../include/b200w4a4.h"
#include "attn_glue.cuh"
#include "gemm_w4a4.cuh"
#include "quant_act.cuh"
#include "weight_pack.cuh"

namespace {

using namespace b200w4a4;

constexpr int kMaxDevices = 64;

// Device status word: kernels write a role code here when a bounded wait runs out.  It is a
// report for the host (b200w4a4_last_device_status / b200w4a4_check_device) and cancels nothing.
__device__ int g_device_status;
// Id of the GEMM launch that last timed out: the other CTAs of that launch, and only they,
// drain early when they see their own id here.
__device__ unsigned g_gemm_abort;

std::atomic<int> g_cta_group{0};  // 0 = not chosen yet (environment decides on first use)
std::atomic<int> g_weight_staging{0};  // 0 = not chosen yet; 4 = packed int4 (default), 8 = int8

struct DeviceState {
  std::once_flag once;
  int err = B200W4A4_OK;
  int sm_count = 0;
  int* status_ptr = nullptr;
  unsigned* abort_ptr = nullptr;
  std::atomic<unsigned> launch_seq{0};
};
DeviceState g_dev[kMaxDevices];

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                   const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                   const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
std::once_flag g_encode_once;
EncodeTiledFn g_encode = nullptr;

EncodeTiledFn get_encode() {
  std::call_once(g_encode_once, [] {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) ==
            cudaSuccess &&
        qres == cudaDriverEntryPointSuccess) {
      g_encode = reinterpret_cast<EncodeTiledFn>(fn);
    }
  });
  return g_encode;
}

template <int CG, int EPI>
bool set_gemm_smem() {
  return cudaFuncSetAttribute(gemm_w4a4_kernel<CG, EPI, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                              GemmCfg<CG, false>::SMEM_ALLOC) == cudaSuccess &&
         cudaFuncSetAttribute(gemm_w4a4_kernel<CG, EPI, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                              GemmCfg<CG, true>::SMEM_ALLOC) == cudaSuccess;
}

// Per-device one-time set-up with that device current: capability check, SM
// count, address of the status word, shared-memory opt-in of the GEMM kernels.
int device_state(DeviceState** out) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return B200W4A4_ECUDA;
  if (dev < 0 || dev >= kMaxDevices) return B200W4A4_EINVAL;
  DeviceState& st = g_dev[dev];
  std::call_once(st.once, [&st, dev] {
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, dev) != cudaSuccess) {
      st.err = B200W4A4_ECUDA;
      return;
    }
    if (prop.major != 10 || prop.minor != 0) {
      st.err = B200W4A4_EARCH;
      return;
    }
    st.sm_count = prop.multiProcessorCount;
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_device_status) != cudaSuccess) {
      st.err = B200W4A4_ECUDA;
      return;
    }
    st.status_ptr = static_cast<int*>(p);
    void* ab = nullptr;
    if (cudaGetSymbolAddress(&ab, g_gemm_abort) != cudaSuccess) {
      st.err = B200W4A4_ECUDA;
      return;
    }
    st.abort_ptr = static_cast<unsigned*>(ab);
    if (cudaMemset(p, 0, sizeof(int)) != cudaSuccess || cudaMemset(ab, 0, sizeof(unsigned)) != cudaSuccess ||
        !set_gemm_smem<1, EPI_NONE>() || !set_gemm_smem<2, EPI_NONE>() ||
        !set_gemm_smem<1, EPI_GELU_TANH>() || !set_gemm_smem<2, EPI_GELU_TANH>() ||
        !set_gemm_smem<1, EPI_GATE_RESIDUAL>() || !set_gemm_smem<2, EPI_GATE_RESIDUAL>() ||
        !set_gemm_smem<1, EPI_SPLIT>() || !set_gemm_smem<2, EPI_SPLIT>()) {
      st.err = B200W4A4_ECUDA;
      return;
    }
  });
  *out = &st;
  return st.err;
}

int current_cta_group() {
  int g = g_cta_group.load(std::memory_order_relaxed);
  if (g == 0) {
    const char* e = getenv("B200W4A4_CTA_GROUP");
    g = (e != nullptr && e[0] == '1') ? 1 : 2;  // the CTA-pair kernel is the default
    g_cta_group.store(g, std::memory_order_relaxed);
  }
  return g;
}

int current_weight_staging() {
  int g = g_weight_staging.load(std::memory_order_relaxed);
  if (g == 0) {
    const char* e = getenv("B200W4A4_WEIGHT_STAGING");
    g = (e != nullptr && (e[0] == '8' || strcmp(e, "int8") == 0)) ? 8 : 4;  // packed int4 is the default
    g_weight_staging.store(g, std::memory_order_relaxed);
  }
  return g;
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

int check_nk(int N, int K) {
  if (N < 128 || K < 64) return B200W4A4_ESHAPE;
  if ((K % 64) != 0 || (N % 128) != 0) return B200W4A4_ESHAPE;
  return B200W4A4_OK;
}

int encode_2d_uncached(CUtensorMap* map, CUtensorMapDataType dt, const void* base, uint64_t inner,
                       uint64_t outer, uint64_t row_stride_bytes, uint32_t box_inner,
                       uint32_t box_outer, CUtensorMapSwizzle sw) {
  EncodeTiledFn enc = get_encode();
  if (enc == nullptr) return B200W4A4_ECUDA;
  const cuuint64_t dims[2] = {inner, outer};
  const cuuint64_t strides[1] = {row_stride_bytes};
  const cuuint32_t box[2] = {box_inner, box_outer};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = enc(map, dt, 2, const_cast<void*>(base), dims, strides, box, estr,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, sw, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? B200W4A4_OK : B200W4A4_ECUDA;
}

// Tensor maps are a pure function of (address, extents, pitch, box, element type, swizzle), and a
// model calls the same layers with the same buffers step after step, so encoded maps are kept
// in a small mutex-guarded table instead of being re-encoded by the driver on every launch.
struct MapKey {
  const void* base;
  uint64_t inner, outer, pitch;
  uint32_t box_inner, box_outer;
  int dt, sw;
  bool operator==(const MapKey& o) const {
    return base == o.base && inner == o.inner && outer == o.outer && pitch == o.pitch &&
           box_inner == o.box_inner && box_outer == o.box_outer && dt == o.dt && sw == o.sw;
  }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    uint64_t h = reinterpret_cast<uintptr_t>(k.base) * 0x9E3779B97F4A7C15ull;
    h ^= (k.inner + 0x9E3779B97F4A7C15ull + (h << 6) + (h >> 2));
    h ^= (k.outer * 0xC2B2AE3D27D4EB4Full + (h << 6) + (h >> 2));
    h ^= (k.pitch + (static_cast<uint64_t>(k.box_outer) << 32) + k.box_inner + (h << 6) + (h >> 2));
    h ^= static_cast<uint64_t>(k.dt * 31 + k.sw);
    return static_cast<size_t>(h);
  }
};
constexpr size_t kMapCacheLimit = 8192;  // entries (128 B each); the table is emptied when full
std::mutex g_map_mutex;
std::unordered_map<MapKey, CUtensorMap, MapKeyHash> g_map_cache;
std::atomic<unsigned long long> g_map_hits{0}, g_map_misses{0};

int encode_2d(CUtensorMap* map, CUtensorMapDataType dt, const void* base, uint64_t inner,
              uint64_t outer, uint64_t row_stride_bytes, uint32_t box_inner, uint32_t box_outer,
              CUtensorMapSwizzle sw) {
  const MapKey key{base, inner, outer, row_stride_bytes, box_inner, box_outer, static_cast<int>(dt),
                   static_cast<int>(sw)};
  {
    std::lock_guard<std::mutex> lock(g_map_mutex);
    auto it = g_map_cache.find(key);
    if (it != g_map_cache.end()) {
      memcpy(map, &it->second, sizeof(CUtensorMap));
      g_map_hits.fetch_add(1, std::memory_order_relaxed);
      return B200W4A4_OK;
    }
  }
  const int rc = encode_2d_uncached(map, dt, base, inner, outer, row_stride_bytes, box_inner, box_outer, sw);
  if (rc != B200W4A4_OK) return rc;
  g_map_misses.fetch_add(1, std::memory_order_relaxed);
  std::lock_guard<std::mutex> lock(g_map_mutex);
  if (g_map_cache.size() >= kMapCacheLimit) g_map_cache.clear();
  g_map_cache.emplace(key, *map);
  return B200W4A4_OK;
}

struct EpiArgs {
  const __half* residual = nullptr;
  const float* gate = nullptr;
  long long gate_row_stride = 0;
  // EPI_SPLIT: `segments` output matrices [M, N / segments] with their own row strides (elements)
  int segments = 0;
  __half* seg_out[3] = {nullptr, nullptr, nullptr};
  long long seg_ld[3] = {0, 0, 0};
};

template <int CG, int EPI, bool W8>
int launch_gemm_staged(DeviceState& st, const void* qact, const float* act_scale, const void* w_b200,
                const __half* w_scale, const __half* bias, __half* out, int32_t* acc_dump, int M,
                int N, int K, cudaStream_t stream, const EpiArgs& epi) {
  using C = GemmCfg<CG, W8>;
  CUtensorMap tm_a, tm_w;
  OutMaps tm_out;
  int rc = encode_2d(&tm_a, CU_TENSOR_MAP_DATA_TYPE_UINT8, qact, static_cast<uint64_t>(K),
                     static_cast<uint64_t>(M), static_cast<uint64_t>(K), C::BK, C::BM,
                     CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc != B200W4A4_OK) return rc;
  if constexpr (W8) {
    rc = encode_2d(&tm_w, CU_TENSOR_MAP_DATA_TYPE_UINT8, w_b200, static_cast<uint64_t>(K),
                   static_cast<uint64_t>(N), static_cast<uint64_t>(K), C::BK, C::B_ROWS,
                   CU_TENSOR_MAP_SWIZZLE_128B);
  } else {
    rc = encode_2d(&tm_w, CU_TENSOR_MAP_DATA_TYPE_UINT8, w_b200, static_cast<uint64_t>(K / 2),
                   static_cast<uint64_t>(N), static_cast<uint64_t>(K / 2), C::BK / 2, C::B_ROWS,
                   CU_TENSOR_MAP_SWIZZLE_NONE);
  }
  if (rc != B200W4A4_OK) return rc;
  if constexpr (EPI == EPI_SPLIT) {
    const int seg_cols = N / epi.segments;
    for (int sg = 0; sg < 3; ++sg) {
      const int src = sg < epi.segments ? sg : 0;  // unused slots repeat segment 0 (never addressed)
      rc = encode_2d(&tm_out.seg[sg], CU_TENSOR_MAP_DATA_TYPE_FLOAT16, epi.seg_out[src],
                     static_cast<uint64_t>(seg_cols), static_cast<uint64_t>(M),
                     static_cast<uint64_t>(epi.seg_ld[src]) * 2, 64, 32, CU_TENSOR_MAP_SWIZZLE_128B);
      if (rc != B200W4A4_OK) return rc;
    }
  } else {
    rc = encode_2d(&tm_out.seg[0], CU_TENSOR_MAP_DATA_TYPE_FLOAT16, out, static_cast<uint64_t>(N),
                   static_cast<uint64_t>(M), static_cast<uint64_t>(N) * 2, 64, 32,
                   CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != B200W4A4_OK) return rc;
    tm_out.seg[1] = tm_out.seg[0];
    tm_out.seg[2] = tm_out.seg[0];
  }

  GemmParams p;
  p.act_scale = act_scale;
  p.w_scale = w_scale;
  p.bias = bias;
  p.acc_dump = acc_dump;
  p.M = M;
  p.N = N;
  p.K = K;
  p.m_tiles = (M + C::BM * CG - 1) / (C::BM * CG);
  p.n_tiles = (N + C::BN - 1) / C::BN;
  p.status = st.status_ptr;
  p.abort_word = st.abort_ptr;
  unsigned id = st.launch_seq.fetch_add(1, std::memory_order_relaxed) + 1;
  if (id == 0) id = st.launch_seq.fetch_add(1, std::memory_order_relaxed) + 1;  // 0 means "no launch"
  p.launch_id = id;
  p.residual = epi.residual;
  p.gate = epi.gate;
  p.gate_row_stride = epi.gate_row_stride;
  p.seg_cols = (EPI == EPI_SPLIT) ? N / epi.segments : N;
  const long long tiles = static_cast<long long>(p.m_tiles) * p.n_tiles;
  const int groups = st.sm_count / CG;
  const unsigned grid = static_cast<unsigned>((tiles < groups ? tiles : groups) * CG);

  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid, 1, 1);
  cfg.blockDim = dim3(C::THREADS, 1, 1);
  cfg.dynamicSmemBytes = C::SMEM_ALLOC;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = CG;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  const cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_w4a4_kernel<CG, EPI, W8>, tm_a, tm_w, tm_out, p);
  return e == cudaSuccess ? B200W4A4_OK : B200W4A4_ECUDA;
}

template <int CG, int EPI = EPI_NONE>
int launch_gemm(DeviceState& st, const void* qact, const float* act_scale, const void* w_b200,
                const __half* w_scale, const __half* bias, __half* out, int32_t* acc_dump, int M,
                int N, int K, cudaStream_t stream, const EpiArgs& epi = EpiArgs()) {
  if (current_weight_staging() == 8)
    return launch_gemm_staged<CG, EPI, true>(st, qact, act_scale, w_b200, w_scale, bias, out, acc_dump, M, N, K,
                                             stream, epi);
  return launch_gemm_staged<CG, EPI, false>(st, qact, act_scale, w_b200, w_scale, bias, out, acc_dump, M, N, K,
                                            stream, epi);
}

// ---- scratch of b200w4a4_linear_noalloc -------------------------------------------------
// Quantised activation codes (int8 [M,K]) followed by the per-token scales (fp32 [M]).
constexpr size_t kNoAllocCodeBytes = static_cast<size_t>(8) << 20;  // M * K <= 8 Mi codes
constexpr int kNoAllocMaxRows = 8192;                               // M <= 8192 tokens
static __device__ __align__(256) uint8_t
    g_noalloc_scratch[kNoAllocCodeBytes + kNoAllocMaxRows * sizeof(float)];

struct NoAllocState {
  std::once_flag once;
  int err = B200W4A4_OK;
  uint8_t* base = nullptr;  // device address of g_noalloc_scratch on this device
};
NoAllocState g_noalloc[kMaxDevices];

// In host code `g_noalloc_scratch` is only a stand-in for the symbol, not a device address:
// the address valid on the current device has to be asked for, once per device.
int noalloc_scratch(uint8_t** base) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return B200W4A4_ECUDA;
  if (dev < 0 || dev >= kMaxDevices) return B200W4A4_EINVAL;
  NoAllocState& st = g_noalloc[dev];
  std::call_once(st.once, [&st] {
    void* ptr = nullptr;
    if (cudaGetSymbolAddress(&ptr, g_noalloc_scratch) != cudaSuccess || ptr == nullptr) {
      cudaGetLastError();
      st.err = B200W4A4_ECUDA;
      return;
    }
    st.base = static_cast<uint8_t*>(ptr);
  });
  *base = st.base;
  return st.err;
}

}  // namespace

extern "C" {

int b200w4a4_version(void) { return B200W4A4_ABI_VERSION; }

const char* b200w4a4_strerror(int code) {
  switch (code) {
    case B200W4A4_OK: return "ok";
    case B200W4A4_EINVAL: return "invalid argument (null pointer, bad size or enum)";
    case B200W4A4_ESHAPE: return "unsupported shape (need K % 64 == 0, N % 128 == 0, M >= 1)";
    case B200W4A4_EALIGN: return "pointer is not 16-byte aligned";
    case B200W4A4_EARCH: return "device is not compute capability 10.0 (sm_100a required)";
    case B200W4A4_ECUDA: return "CUDA runtime or driver call failed";
    case B200W4A4_EWORKSPACE: return "workspace too small";
    case B200W4A4_EDEVICE: return "a kernel recorded a device-side time-out";
    case B200W4A4_ELIMIT: return "activation too large for the built-in scratch of the no-alloc entry point";
    default: return "unknown b200w4a4 error code";
  }
}

int b200w4a4_query(int device, int* sm_count, int* cc_major, int* cc_minor) {
  cudaDeviceProp prop;
  if (cudaGetDeviceProperties(&prop, device) != cudaSuccess) {
    cudaGetLastError();
    return B200W4A4_ECUDA;
  }
  if (sm_count != nullptr) *sm_count = prop.multiProcessorCount;
  if (cc_major != nullptr) *cc_major = prop.major;
  if (cc_minor != nullptr) *cc_minor = prop.minor;
  return (prop.major == 10 && prop.minor == 0) ? B200W4A4_OK : B200W4A4_EARCH;
}

int b200w4a4_pack_weight(const void* w_f16, const void* ch_scale_f16, void* vdm_packed,
                         void* vdm_scale_packed, void* vdm_scale, int N, int K, void* stream) {
  if (w_f16 == nullptr || vdm_packed == nullptr || vdm_scale_packed == nullptr ||
      vdm_scale == nullptr)
    return B200W4A4_EINVAL;
  int rc = check_nk(N, K);
  if (rc != B200W4A4_OK) return rc;
  if (!aligned16(w_f16) || !aligned16(vdm_packed)) return B200W4A4_EALIGN;
  DeviceState* st = nullptr;
  if ((rc = device_state(&st)) != B200W4A4_OK) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const __half* w = static_cast<const __half*>(w_f16);
  const __half* scale = static_cast<const __half*>(ch_scale_f16);
  if (scale == nullptr) {
    weight_absmax_scale_kernel<<<static_cast<unsigned>(N), 256, 0, s>>>(
        w, static_cast<__half*>(vdm_scale), N, K);
    scale = static_cast<const __half*>(vdm_scale);
  }
  const size_t words = static_cast<size_t>(N) * K / 8;
  pack_weight_v1_kernel<<<static_cast<unsigned>((words + 255) / 256), 256, 0, s>>>(
      w, scale, static_cast<uint32_t*>(vdm_packed), N, K);
  const size_t nscale = static_cast<size_t>(N) * (K / 64);
  pack_wscale_v1_kernel<<<static_cast<unsigned>((nscale + 255) / 256), 256, 0, s>>>(
      scale, static_cast<__half*>(vdm_scale_packed),
      static_cast<const void*>(scale) == vdm_scale ? nullptr : static_cast<__half*>(vdm_scale), N, K);
  return cudaGetLastError() == cudaSuccess ? B200W4A4_OK : B200W4A4_ECUDA;
}

size_t b200w4a4_repack_bytes(int N, int K) {
  if (check_nk(N, K) != B200W4A4_OK) return 0;
  return current_weight_staging() == 8 ? static_cast<size_t>(N) * K : static_cast<size_t>(N) * (K / 2);
}

int b200w4a4_repack_weight(const void* vdm_packed, void* w_b200, const void* vdm_scale_packed,
                           void* w_scale_plain, int N, int K, void* stream) {
  if (vdm_packed == nullptr || w_b200 == nullptr) return B200W4A4_EINVAL;
  if ((vdm_scale_packed == nullptr) != (w_scale_plain == nullptr)) return B200W4A4_EINVAL;
  int rc = check_nk(N, K);
  if (rc != B200W4A4_OK) return rc;
  if (!aligned16(vdm_packed) || !aligned16(w_b200)) return B200W4A4_EALIGN;
  DeviceState* st = nullptr;
  if ((rc = device_state(&st)) != B200W4A4_OK) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (current_weight_staging() == 8) {
    const size_t words = static_cast<size_t>(N) * (K / 8);
    expand_v1_to_int8_kernel<<<static_cast<unsigned>((words + 255) / 256), 256, 0, s>>>(
        static_cast<const uint32_t*>(vdm_packed), static_cast<uint2*>(w_b200), N, K);
  } else {
    const size_t chunks = static_cast<size_t>(N) * (K / 32);
    repack_v1_to_b200_kernel<<<static_cast<unsigned>((chunks + 255) / 256), 256, 0, s>>>(
        static_cast<const uint32_t*>(vdm_packed), static_cast<uint4*>(w_b200), N, K);
  }
  if (vdm_scale_packed != nullptr) {
    unswizzle_wscale_v1_kernel<<<static_cast<unsigned>((N + 255) / 256), 256, 0, s>>>(
        static_cast<const __half*>(vdm_scale_packed), static_cast<__half*>(w_scale_plain), N, K);
  }
  return cudaGetLastError() == cudaSuccess ? B200W4A4_OK : B200W4A4_ECUDA;
}

size_t b200w4a4_qact_bytes(int M, int K, int container) {
  if (M < 1 || K < 64 || (K % 64) != 0) return 0;
  if (container == B200W4A4_QACT_INT8) return static_cast<size_t>(M) * K;
  if (container == B200W4A4_QACT_NIBBLE) return static_cast<size_t>(M) * (K / 2);
  return 0;
}

int b200w4a4_quantize_act(const void* x, int x_dtype, void* qact, int container, float* act_scale,
                          int M, int K, float clip, void* stream) {
  if (x == nullptr || qact == nullptr || act_scale == nullptr) return B200W4A4_EINVAL;
  if (M < 1 || K < 64 || (K % 64) != 0) return B200W4A4_ESHAPE;
  if (!(clip > 0.0f)) return B200W4A4_EINVAL;
  if (!aligned16(x) || !aligned16(qact)) return B200W4A4_EALIGN;
  DeviceState* st = nullptr;
  int rc = device_state(&st);
  if (rc != B200W4A4_OK) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  cudaError_t e = cudaErrorInvalidValue;
#define B200W4A4_QDISPATCH(T)                                                                     \
  (container == B200W4A4_QACT_INT8                                                                \
       ? launch_quant_act<T, QOUT_INT8>(static_cast<const T*>(x), qact, act_scale, M, K, clip, s) \
       : launch_quant_act<T, QOUT_NIBBLE>(static_cast<const T*>(x), qact, act_scale, M, K, clip, s))
  if (container != B200W4A4_QACT_INT8 && container != B200W4A4_QACT_NIBBLE) return B200W4A4_EINVAL;
  switch (x_dtype) {
    case B200W4A4_F16: e = B200W4A4_QDISPATCH(__half); break;
    case B200W4A4_BF16: e = B200W4A4_QDISPATCH(__nv_bfloat16); break;
    case B200W4A4_F32: e = B200W4A4_QDISPATCH(float); break;
    default: return B200W4A4_EINVAL;
  }
#undef B200W4A4_QDISPATCH
  return e == cudaSuccess ? B200W4A4_OK : B200W4A4_ECUDA;
}

int b200w4a4_gemm(const void* qact, const float* act_scale, const void* w_b200, const void* w_scale,
                  const void* bias, void* out, int32_t* acc_dump, int M, int N, int K,
                  void* stream) {
  if (qact == nullptr || act_scale == nullptr || w_b200 == nullptr || w_scale == nullptr ||
      out == nullptr)
    return B200W4A4_EINVAL;
  if (M < 1) return B200W4A4_ESHAPE;
  int rc = check_nk(N, K);
  if (rc != B200W4A4_OK) return rc;
  if (!aligned16(qact) || !aligned16(w_b200) || !aligned16(w_scale) || !aligned16(out) ||
      (bias != nullptr && !aligned16(bias)) || (acc_dump != nullptr && !aligned16(acc_dump)))
    return B200W4A4_EALIGN;
  DeviceState* st = nullptr;
  if ((rc = device_state(&st)) != B200W4A4_OK) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (current_cta_group() == 2)
    return launch_gemm<2>(*st, qact, act_scale, w_b200, static_cast<const __half*>(w_scale),
                          static_cast<const __half*>(bias), static_cast<__half*>(out), acc_dump, M,
                          N, K, s);
  return launch_gemm<1>(*st, qact, act_scale, w_b200, static_cast<const __half*>(w_scale),
                        static_cast<const __half*>(bias), static_cast<__half*>(out), acc_dump, M, N,
                        K, s);
}

size_t b200w4a4_linear_workspace_bytes(int M, int K) {
  if (M < 1 || K < 64 || (K % 64) != 0) return 0;
  const size_t codes = (static_cast<size_t>(M) * K + 255) & ~static_cast<size_t>(255);
  const size_t scales = (static_cast<size_t>(M) * sizeof(float) + 255) & ~static_cast<size_t>(255);
  return codes + scales;
}

int b200w4a4_linear(const void* x, int x_dtype, const void* w_b200, const void* w_scale,
                    const void* bias, void* out, void* workspace, size_t workspace_bytes, int M,
                    int N, int K, float clip, void* stream) {
  if (workspace == nullptr) return B200W4A4_EINVAL;
  const size_t need = b200w4a4_linear_workspace_bytes(M, K);
  if (need == 0) return B200W4A4_ESHAPE;
  if (workspace_bytes < need) return B200W4A4_EWORKSPACE;
  if ((reinterpret_cast<uintptr_t>(workspace) & 255u) != 0) return B200W4A4_EALIGN;
  uint8_t* ws = static_cast<uint8_t*>(workspace);
  void* qact = ws;
  float* act_scale =
      reinterpret_cast<float*>(ws + ((static_cast<size_t>(M) * K + 255) & ~static_cast<size_t>(255)));
  int rc = b200w4a4_quantize_act(x, x_dtype, qact, B200W4A4_QACT_INT8, act_scale, M, K, clip, stream);
  if (rc != B200W4A4_OK) return rc;
  return b200w4a4_gemm(qact, act_scale, w_b200, w_scale, bias, out, nullptr, M, N, K, stream);
}

// ---- fused variants ------------------------------------------------------------------
int b200w4a4_quantize_act_fused(const void* x_f16, int prologue, const float* mod_scale,
                                const float* mod_shift, long long mod_row_stride, float ln_eps,
                                void* qact, float* act_scale, int M, int K, float clip,
                                void* stream) {
  if (x_f16 == nullptr || qact == nullptr || act_scale == nullptr) return B200W4A4_EINVAL;
  if (M < 1 || K < 64 || (K % 64) != 0 || K > 16384) return B200W4A4_ESHAPE;
  if (!(clip > 0.0f)) return B200W4A4_EINVAL;
  if (!aligned16(x_f16) || !aligned16(qact)) return B200W4A4_EALIGN;
  if (prologue == B200W4A4_PRE_NONE)
    return b200w4a4_quantize_act(x_f16, B200W4A4_F16, qact, B200W4A4_QACT_INT8, act_scale, M, K, clip,
                                 stream);
  DeviceState* st = nullptr;
  int rc = device_state(&st);
  if (rc != B200W4A4_OK) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  PreArgs pre;
  pre.mod_scale = mod_scale;
  pre.mod_shift = mod_shift;
  pre.mod_row_stride = mod_row_stride;
  pre.ln_eps = ln_eps;
  cudaError_t e;
  if (prologue == B200W4A4_PRE_GELU_TANH) {
    e = launch_quant_act_pre<PRE_GELU_TANH>(static_cast<const __half*>(x_f16), qact, act_scale, M, K,
                                            clip, pre, s);
  } else if (prologue == B200W4A4_PRE_LAYERNORM_MOD) {
    if (mod_scale == nullptr || mod_shift == nullptr) return B200W4A4_EINVAL;
    if (!aligned16(mod_scale) || !aligned16(mod_shift) || (mod_row_stride % 4) != 0)
      return B200W4A4_EALIGN;
    e = launch_quant_act_pre<PRE_LAYERNORM_MOD>(static_cast<const __half*>(x_f16), qact, act_scale, M,
                                                K, clip, pre, s);
  } else {
    return B200W4A4_EINVAL;
  }
  return e == cudaSuccess ? B200W4A4_OK : B200W4A4_ECUDA;
}

int b200w4a4_gemm_fused(const void* qact, const float* act_scale, const void* w_b200,
                        const void* w_scale, const void* bias, void* out, int epilogue,
                        const void* residual_f16, const float* gate, long long gate_row_stride, int M,
                        int N, int K, void* stream) {
  if (epilogue == B200W4A4_EPI_NONE)
    return b200w4a4_gemm(qact, act_scale, w_b200, w_scale, bias, out, nullptr, M, N, K, stream);
  if (qact == nullptr || act_scale == nullptr || w_b200 == nullptr || w_scale == nullptr ||
      out == nullptr)
    return B200W4A4_EINVAL;
  if (M < 1) return B200W4A4_ESHAPE;
  int rc = check_nk(N, K);
  if (rc != B200W4A4_OK) return rc;
  if (!aligned16(qact) || !aligned16(w_b200) || !aligned16(w_scale) || !aligned16(out) ||
      (bias != nullptr && !aligned16(bias)))
    return B200W4A4_EALIGN;
  EpiArgs epi;
  if (epilogue == B200W4A4_EPI_GATE_RESIDUAL) {
    if (residual_f16 == nullptr || gate == nullptr) return B200W4A4_EINVAL;
    if (!aligned16(residual_f16) || !aligned16(gate) || (gate_row_stride % 4) != 0)
      return B200W4A4_EALIGN;
    epi.residual = static_cast<const __half*>(residual_f16);
    epi.gate = gate;
    epi.gate_row_stride = gate_row_stride;
  } else if (epilogue != B200W4A4_EPI_GELU_TANH) {
    return B200W4A4_EINVAL;
  }
  DeviceState* st = nullptr;
  if ((rc = device_state(&st)) != B200W4A4_OK) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const __half* ws = static_cast<const __half*>(w_scale);
  const __half* b = static_cast<const __half*>(bias);
  __half* o = static_cast<__half*>(out);
  const bool pair = current_cta_group() == 2;
  if (epilogue == B200W4A4_EPI_GELU_TANH)
    return pair ? launch_gemm<2, EPI_GELU_TANH>(*st, qact, act_scale, w_b200, ws, b, o, nullptr, M, N, K, s, epi)
                : launch_gemm<1, EPI_GELU_TANH>(*st, qact, act_scale, w_b200, ws, b, o, nullptr, M, N, K, s, epi);
  return pair ? launch_gemm<2, EPI_GATE_RESIDUAL>(*st, qact, act_scale, w_b200, ws, b, o, nullptr, M, N, K, s, epi)
              : launch_gemm<1, EPI_GATE_RESIDUAL>(*st, qact, act_scale, w_b200, ws, b, o, nullptr, M, N, K, s, epi);
}

int b200w4a4_gemm_split(const void* qact, const float* act_scale, const void* w_b200,
                        const void* w_scale, const void* bias, void* const* outs,
                        const long long* out_ld, int segments, int M, int N, int K, void* stream) {
  if (qact == nullptr || act_scale == nullptr || w_b200 == nullptr || w_scale == nullptr ||
      outs == nullptr || out_ld == nullptr)
    return B200W4A4_EINVAL;
  if (segments < 1 || segments > 3) return B200W4A4_EINVAL;
  if (M < 1) return B200W4A4_ESHAPE;
  int rc = check_nk(N, K);
  if (rc != B200W4A4_OK) return rc;
  if ((N % segments) != 0 || ((N / segments) % 64) != 0) return B200W4A4_ESHAPE;
  if (!aligned16(qact) || !aligned16(w_b200) || !aligned16(w_scale) ||
      (bias != nullptr && !aligned16(bias)))
    return B200W4A4_EALIGN;
  EpiArgs epi;
  epi.segments = segments;
  for (int sg = 0; sg < segments; ++sg) {
    if (outs[sg] == nullptr) return B200W4A4_EINVAL;
    if (out_ld[sg] < N / segments) return B200W4A4_ESHAPE;
    // the tensor map wants a 16-byte aligned base and row pitch
    if (!aligned16(outs[sg]) || (out_ld[sg] % 8) != 0) return B200W4A4_EALIGN;
    epi.seg_out[sg] = static_cast<__half*>(outs[sg]);
    epi.seg_ld[sg] = out_ld[sg];
  }
  DeviceState* st = nullptr;
  if ((rc = device_state(&st)) != B200W4A4_OK) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const __half* ws = static_cast<const __half*>(w_scale);
  const __half* b = static_cast<const __half*>(bias);
  return current_cta_group() == 2
             ? launch_gemm<2, EPI_SPLIT>(*st, qact, act_scale, w_b200, ws, b, nullptr, nullptr, M, N, K, s, epi)
             : launch_gemm<1, EPI_SPLIT>(*st, qact, act_scale, w_b200, ws, b, nullptr, nullptr, M, N, K, s, epi);
}

int b200w4a4_qk_norm_rope_push(const void* x_f16, long long x_ld, const void* norm_weight_f16,
                               const float* rope_cos_sin, float eps, int head_dim, void* const* outs,
                               int n_outs, int out_dtype, long long out_ld, long long out_row0,
                               uint32_t* const* flags, int flag_index, uint32_t epoch,
                               unsigned int* ticket, int L, int D, void* stream) {
  if (x_f16 == nullptr || outs == nullptr) return B200W4A4_EINVAL;
  if (n_outs < 1 || n_outs > kMaxPushDestinations || out_row0 < 0 || flag_index < 0)
    return B200W4A4_EINVAL;
  if ((flags != nullptr) != (ticket != nullptr)) return B200W4A4_EINVAL;
  if (out_dtype != B200W4A4_F16 && out_dtype != B200W4A4_BF16) return B200W4A4_EINVAL;
  if (L < 1 || D < 8 || (D % 8) != 0 || D > 16384 || x_ld < D || out_ld < D) return B200W4A4_ESHAPE;
  if (rope_cos_sin != nullptr && (head_dim < 8 || (head_dim % 8) != 0 || (D % head_dim) != 0))
    return B200W4A4_ESHAPE;
  if (!aligned16(x_f16) || (x_ld % 8) != 0 || (out_ld % 8) != 0 ||
      (norm_weight_f16 != nullptr && !aligned16(norm_weight_f16)) ||
      (rope_cos_sin != nullptr && !aligned16(rope_cos_sin)))
    return B200W4A4_EALIGN;
  QkNormRopeArgs a;
  for (int d = 0; d < kMaxPushDestinations; ++d) {
    a.out[d] = nullptr;
    a.flag[d] = nullptr;
  }
  for (int d = 0; d < n_outs; ++d) {
    if (outs[d] == nullptr) return B200W4A4_EINVAL;
    if (!aligned16(outs[d])) return B200W4A4_EALIGN;
    a.out[d] = outs[d];
    if (flags != nullptr) a.flag[d] = flags[d];  // a null entry: no signal for that destination
  }
  DeviceState* st = nullptr;
  const int rc = device_state(&st);
  if (rc != B200W4A4_OK) return rc;
  a.x = static_cast<const __half*>(x_f16);
  a.x_ld = x_ld;
  a.weight = static_cast<const __half*>(norm_weight_f16);
  a.cos_sin = rope_cos_sin;
  a.eps = eps;
  a.head_dim = head_dim;
  a.n_out = n_outs;
  a.out_ld = out_ld;
  a.out_row0 = out_row0;
  a.flag_index = flag_index;
  a.epoch = epoch;
  a.ticket = ticket;
  a.L = L;
  a.D = D;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const bool push = n_outs > 1 || ticket != nullptr;
  cudaError_t e;
  if (out_dtype == B200W4A4_BF16)
    e = push ? launch_qk_norm_rope<true, true>(a, s) : launch_qk_norm_rope<true, false>(a, s);
  else
    e = push ? launch_qk_norm_rope<false, true>(a, s) : launch_qk_norm_rope<false, false>(a, s);
  return e == cudaSuccess ? B200W4A4_OK : B200W4A4_ECUDA;
}

int b200w4a4_qk_norm_rope(const void* x_f16, long long x_ld, const void* norm_weight_f16,
                          const float* rope_cos_sin, float eps, int head_dim, void* out, int out_dtype,
                          long long out_ld, int L, int D, void* stream) {
  if (out == nullptr) return B200W4A4_EINVAL;
  void* outs[1] = {out};
  return b200w4a4_qk_norm_rope_push(x_f16, x_ld, norm_weight_f16, rope_cos_sin, eps, head_dim, outs, 1,
                                    out_dtype, out_ld, 0, nullptr, 0, 0u, nullptr, L, D, stream);
}

int b200w4a4_attn_merge(const void* o1_bf16, long long o1_ld, const void* o2_bf16, long long o2_ld,
                        const float* lse1, const float* lse2, void* out_bf16, int L, int H, int head_dim,
                        void* stream) {
  if (o1_bf16 == nullptr || o2_bf16 == nullptr || lse1 == nullptr || lse2 == nullptr || out_bf16 == nullptr)
    return B200W4A4_EINVAL;
  if (L < 1 || H < 1 || head_dim < 8 || (head_dim % 8) != 0) return B200W4A4_ESHAPE;
  const long long d = static_cast<long long>(H) * head_dim;
  if (o1_ld < d || o2_ld < d) return B200W4A4_ESHAPE;
  if (!aligned16(o1_bf16) || !aligned16(o2_bf16) || !aligned16(out_bf16) || (o1_ld % 8) != 0 || (o2_ld % 8) != 0)
    return B200W4A4_EALIGN;
  DeviceState* st = nullptr;
  const int rc = device_state(&st);
  if (rc != B200W4A4_OK) return rc;
  const long long threads = static_cast<long long>(L) * (d / 8);
  attn_merge_kernel<<<static_cast<unsigned>((threads + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(o1_bf16), static_cast<const __nv_bfloat16*>(o2_bf16), lse1, lse2,
      static_cast<__nv_bfloat16*>(out_bf16), L, H, head_dim, o1_ld, o2_ld);
  return cudaGetLastError() == cudaSuccess ? B200W4A4_OK : B200W4A4_ECUDA;
}

int b200w4a4_wait_flags(const uint32_t* flags, int n, uint32_t epoch, int timeout_ms, void* stream) {
  if (flags == nullptr || n < 1 || n > 32 || timeout_ms < 1 || timeout_ms > 10000) return B200W4A4_EINVAL;
  DeviceState* st = nullptr;
  const int rc = device_state(&st);
  if (rc != B200W4A4_OK) return rc;
  wait_flags_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(
      flags, n, epoch, static_cast<unsigned long long>(timeout_ms) * 1000000ull, st->status_ptr);
  return cudaGetLastError() == cudaSuccess ? B200W4A4_OK : B200W4A4_ECUDA;
}

int b200w4a4_signal_flags(uint32_t* const* flags, int n, int index, uint32_t value, void* stream) {
  if (flags == nullptr || n < 1 || n > kMaxPushDestinations || index < 0) return B200W4A4_EINVAL;
  DeviceState* st = nullptr;
  const int rc = device_state(&st);
  if (rc != B200W4A4_OK) return rc;
  SignalArgs a;
  for (int d = 0; d < kMaxPushDestinations; ++d) a.flag[d] = d < n ? flags[d] : nullptr;
  a.n = n;
  a.index = index;
  a.value = value;
  signal_flags_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(a);
  return cudaGetLastError() == cudaSuccess ? B200W4A4_OK : B200W4A4_ECUDA;
}

int b200w4a4_linear_fused(const void* x_f16, int prologue, const float* mod_scale,
                          const float* mod_shift, long long mod_row_stride, float ln_eps,
                          const void* w_b200, const void* w_scale, const void* bias, void* out,
                          int epilogue, const void* residual_f16, const float* gate,
                          long long gate_row_stride, void* workspace, size_t workspace_bytes, int M,
                          int N, int K, float clip, void* stream) {
  if (workspace == nullptr) return B200W4A4_EINVAL;
  const size_t need = b200w4a4_linear_workspace_bytes(M, K);
  if (need == 0) return B200W4A4_ESHAPE;
  if (workspace_bytes < need) return B200W4A4_EWORKSPACE;
  if ((reinterpret_cast<uintptr_t>(workspace) & 255u) != 0) return B200W4A4_EALIGN;
  uint8_t* wsp = static_cast<uint8_t*>(workspace);
  float* act_scale =
      reinterpret_cast<float*>(wsp + ((static_cast<size_t>(M) * K + 255) & ~static_cast<size_t>(255)));
  int rc = b200w4a4_quantize_act_fused(x_f16, prologue, mod_scale, mod_shift, mod_row_stride, ln_eps,
                                       wsp, act_scale, M, K, clip, stream);
  if (rc != B200W4A4_OK) return rc;
  return b200w4a4_gemm_fused(wsp, act_scale, w_b200, w_scale, bias, out, epilogue, residual_f16, gate,
                             gate_row_stride, M, N, K, stream);
}

size_t b200w4a4_linear_noalloc_max_codes(void) { return kNoAllocCodeBytes; }

int b200w4a4_linear_noalloc_max_rows(void) { return kNoAllocMaxRows; }

// Quantise + GEMM with the intermediate codes and scales held in a device array that is part
// of the library image, for callers that must not allocate device memory at all.
int b200w4a4_linear_noalloc(const void* x, int x_dtype, const void* w_b200, const void* w_scale,
                            const void* bias, void* out, int M, int N, int K, float clip,
                            void* stream) {
  if (M < 1 || K < 64 || (K % 64) != 0) return B200W4A4_ESHAPE;
  if (M > kNoAllocMaxRows || static_cast<size_t>(M) * static_cast<size_t>(K) > kNoAllocCodeBytes)
    return B200W4A4_ELIMIT;
  DeviceState* st = nullptr;
  int rc = device_state(&st);  // a device that is not 10.0 answers EARCH before any symbol look-up
  if (rc != B200W4A4_OK) return rc;
  uint8_t* base = nullptr;
  rc = noalloc_scratch(&base);
  if (rc != B200W4A4_OK) return rc;
  void* qact = base;
  float* act_scale = reinterpret_cast<float*>(base + kNoAllocCodeBytes);
  // Nothing in the scratch has to start at zero: the quantiser rewrites codes [M,K] and scales
  // [M] before the GEMM reads them, and the GEMM's tensor map ends at row M.
  rc = b200w4a4_quantize_act(x, x_dtype, qact, B200W4A4_QACT_INT8, act_scale, M, K, clip, stream);
  if (rc != B200W4A4_OK) return rc;
  return b200w4a4_gemm(qact, act_scale, w_b200, w_scale, bias, out, nullptr, M, N, K, stream);
}

int b200w4a4_unpack_codes(const void* packed, int8_t* codes, int rows, int K, int which,
                          void* stream) {
  if (packed == nullptr || codes == nullptr) return B200W4A4_EINVAL;
  if (rows < 1 || K < 64 || (K % 64) != 0) return B200W4A4_ESHAPE;
  DeviceState* st = nullptr;
  int rc = device_state(&st);
  if (rc != B200W4A4_OK) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const size_t total = static_cast<size_t>(rows) * K;
  const unsigned grid = static_cast<unsigned>((total + 255) / 256);
  switch (which) {
    case B200W4A4_CODES_WEIGHT_B200:
      if (current_weight_staging() == 8)
        unpack_int8_weight_kernel<<<grid, 256, 0, s>>>(static_cast<const int8_t*>(packed), codes, rows, K);
      else
        unpack_b200_weight_kernel<<<grid, 256, 0, s>>>(static_cast<const uint8_t*>(packed), codes,
                                                       rows, K);
      break;
    case B200W4A4_CODES_WEIGHT_V1:
      if ((rows % 128) != 0) return B200W4A4_ESHAPE;
      unpack_v1_weight_kernel<<<grid, 256, 0, s>>>(static_cast<const uint32_t*>(packed), codes, rows,
                                                   K);
      break;
    case B200W4A4_CODES_ACT_NIBBLE:
      unpack_nibble_rows_kernel<<<grid, 256, 0, s>>>(static_cast<const uint8_t*>(packed), codes,
                                                     rows, K);
      break;
    default:
      return B200W4A4_EINVAL;
  }
  return cudaGetLastError() == cudaSuccess ? B200W4A4_OK : B200W4A4_ECUDA;
}

int b200w4a4_set_cta_group(int cta_group) {
  if (cta_group != 1 && cta_group != 2) return B200W4A4_EINVAL;
  const int prev = current_cta_group();
  g_cta_group.store(cta_group, std::memory_order_relaxed);
  return prev;
}

void b200w4a4_map_cache_stats(unsigned long long* hits, unsigned long long* misses) {
  if (hits != nullptr) *hits = g_map_hits.load(std::memory_order_relaxed);
  if (misses != nullptr) *misses = g_map_misses.load(std::memory_order_relaxed);
}

int b200w4a4_check_device(int device) {
  int prev = 0;
  if (cudaGetDevice(&prev) != cudaSuccess) return B200W4A4_ECUDA;
  if (cudaSetDevice(device) != cudaSuccess) {
    cudaGetLastError();
    return B200W4A4_ECUDA;
  }
  DeviceState* st = nullptr;
  int rc = device_state(&st);
  if (rc == B200W4A4_OK) {
    int value = 0;
    if (cudaDeviceSynchronize() != cudaSuccess ||
        cudaMemcpy(&value, st->status_ptr, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess)
      rc = B200W4A4_ECUDA;
    else if (value != 0)
      rc = B200W4A4_EDEVICE;  // the code itself stays readable through b200w4a4_last_device_status
  }
  cudaSetDevice(prev);
  return rc;
}

int b200w4a4_set_weight_staging(int bits) {
  if (bits != 0 && bits != 4 && bits != 8) return B200W4A4_EINVAL;
  const int prev = current_weight_staging();
  if (bits != 0) g_weight_staging.store(bits, std::memory_order_relaxed);
  return prev;
}

int b200w4a4_last_device_status(int device) {
  int prev = 0;
  if (cudaGetDevice(&prev) != cudaSuccess) return B200W4A4_ECUDA;
  if (cudaSetDevice(device) != cudaSuccess) {
    cudaGetLastError();
    return B200W4A4_ECUDA;
  }
  int rc = B200W4A4_OK;
  DeviceState* st = nullptr;
  rc = device_state(&st);
  int value = 0;
  if (rc == B200W4A4_OK) {
    if (cudaDeviceSynchronize() != cudaSuccess ||
        cudaMemcpy(&value, st->status_ptr, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess ||
        cudaMemset(st->status_ptr, 0, sizeof(int)) != cudaSuccess)
      rc = B200W4A4_ECUDA;
  }
  cudaSetDevice(prev);
  return rc == B200W4A4_OK ? value : rc;
}

}  // extern "C"
