/*
 * b200w4a4 -- C ABI of the sm_100a W4A4 linear-layer library.
 *
 * Every entry point takes plain device pointers, sizes and a CUDA stream
 * (passed as void*, i.e. a cudaStream_t; NULL = legacy default stream),
 * launches asynchronously on that stream, allocates nothing, and returns
 * 0 on success or a negative B200W4A4_E* code.  The caller owns all buffers.
 * Shape constraints kept from the reference extension
 * (vdm_infer/kernels/csrc/vdm_w4a4_kernel.cu:769-789): K % 64 == 0,
 * N % 128 == 0, M >= 1 arbitrary (no padding to 256 rows is needed).
 *
 * Each declaration cites the reference interface it stands in for
 * (paths relative to the DSAQuant repository root).
 */
#ifndef B200W4A4_H_
#define B200W4A4_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B200W4A4_ABI_VERSION 1

/* error codes */
#define B200W4A4_OK 0
#define B200W4A4_EINVAL (-1)      /* null pointer, bad size, bad enum */
#define B200W4A4_ESHAPE (-2)      /* K % 64 != 0, N % 128 != 0, M < 1, ... */
#define B200W4A4_EALIGN (-3)      /* pointer not 16-byte aligned */
#define B200W4A4_EARCH (-4)       /* device is not compute capability 10.0 */
#define B200W4A4_ECUDA (-5)       /* CUDA runtime / driver call failed */
#define B200W4A4_EWORKSPACE (-6)  /* workspace too small */
#define B200W4A4_EDEVICE (-7)     /* a kernel recorded a device-side time-out */
#define B200W4A4_ELIMIT (-8)      /* beyond the built-in scratch of b200w4a4_linear_noalloc */

/* activation dtypes accepted by the quantiser */
#define B200W4A4_F16 0
#define B200W4A4_BF16 1
#define B200W4A4_F32 2

/* containers for activation codes */
#define B200W4A4_QACT_INT8 0    /* int8 [M,K], one code per byte (GEMM input) */
#define B200W4A4_QACT_NIBBLE 1  /* u8 [M,K/2], code 2b low nibble, 2b+1 high nibble */

/* `which` of b200w4a4_unpack_codes */
#define B200W4A4_CODES_WEIGHT_B200 1  /* repacked weight  -> int8 [N,K] */
#define B200W4A4_CODES_WEIGHT_V1 2    /* vdm_weight_packed -> int8 [N,K] */
#define B200W4A4_CODES_ACT_NIBBLE 3   /* nibble activations -> int8 [M,K] */

/* ABI version of the loaded library (compare with B200W4A4_ABI_VERSION). */
int b200w4a4_version(void);

/* Human-readable text for an error code.  Never NULL. */
const char* b200w4a4_strerror(int code);

/* Device properties; returns B200W4A4_EARCH unless the device is 10.0.
 * Stands in for the JIT arch selection of vdm_infer/kernels/vdm_w4a4.py:42-69,
 * which gains the sm_100a target. */
int b200w4a4_query(int device, int* sm_count, int* cc_major, int* cc_minor);

/* ---- weights (load / export time) --------------------------------------- */

/* fp16 weight [N,K] + per-channel fp16 scale [N] -> the three buffers of the
 * vdm_w4a4_packed_v1 format: vdm_packed u8 [N,K/2], vdm_scale_packed f16 [N,K/64],
 * vdm_scale f16 [N].  Replaces ext.pack_weight_with_scale
 * (vdm_w4a4_kernel.cu:697-728; python vdm_w4a4.py:209-214).
 * If ch_scale is NULL the scale is computed as absmax/7 per channel into
 * vdm_scale first: ext.quantize_weight_per_channel (vdm_w4a4_kernel.cu:730-763;
 * vdm_w4a4.py:217-219). */
int b200w4a4_pack_weight(const void* w_f16, const void* ch_scale_f16, void* vdm_packed,
                         void* vdm_scale_packed, void* vdm_scale, int N, int K, void* stream);

/* Bytes of the tcgen05-friendly weight buffer for an [N,K] layer. */
size_t b200w4a4_repack_bytes(int N, int K);

/* Load-time repack: vdm_weight_packed (v1 fragment order) -> row-major nibble
 * layout staged by TMA; optionally vdm_weight_scale_packed [N,K/64] -> plain
 * per-channel scale [N] (pass NULLs to skip).  Hooks in where
 * load_packed_quantized_model registers the buffers
 * (vdm_infer/checkpoints/packed_checkpoint.py:52-148). */
int b200w4a4_repack_weight(const void* vdm_packed, void* w_b200, const void* vdm_scale_packed,
                           void* w_scale_plain, int N, int K, void* stream);

/* ---- activations -------------------------------------------------------- */

/* Bytes of the code buffer for M x K activations in the given container. */
size_t b200w4a4_qact_bytes(int M, int K, int container);

/* Dynamic per-token int4 quantise: x [M,K] row-major (ld = K) of dtype
 * x_dtype -> codes in `container`, fp32 scale [M].
 * scale = (max(absmax,1e-5)/7)*clip, code = clamp(rint(x/scale),-8,7).
 * Replaces token_scale_kernel + act_quantize_per_token_kernel
 * (vdm_w4a4_kernel.cu:459-516) / ext.quantize_activation_per_token (:840-873). */
int b200w4a4_quantize_act(const void* x, int x_dtype, void* qact, int container, float* act_scale,
                          int M, int K, float clip, void* stream);

/* ---- GEMM --------------------------------------------------------------- */

/* out[m,n] = fp16( float(sum_k qa[m,k]*qw[n,k]) * (act_scale[m]*w_scale[n]) + bias[n] )
 * qact: int8 container [M,K]; w_b200: repacked weight; w_scale f16 [N];
 * bias f16 [N] or NULL; out f16 [M,N] (ld = N); acc_dump int32 [M,N] or NULL
 * (exact accumulators, for tests).  Replaces linear_w4a4_kernel
 * (vdm_w4a4_kernel.cu:627-686) / ext.linear_prequantized (:876-918). */
int b200w4a4_gemm(const void* qact, const float* act_scale, const void* w_b200, const void* w_scale,
                  const void* bias, void* out, int32_t* acc_dump, int M, int N, int K,
                  void* stream);

/* Workspace bytes b200w4a4_linear needs for an M x K activation. */
size_t b200w4a4_linear_workspace_bytes(int M, int K);

/* Quantise + GEMM: what QuantLinear.forward and the fused QKV projection call.
 * Replaces ext.linear_dynamic / ext.linear_dynamic_bias
 * (vdm_w4a4_kernel.cu:765-838; python linear_vdm_w4a4, vdm_w4a4.py:222-244). */
int b200w4a4_linear(const void* x, int x_dtype, const void* w_b200, const void* w_scale,
                    const void* bias, void* out, void* workspace, size_t workspace_bytes, int M,
                    int N, int K, float clip, void* stream);

/* ---- fused variants ------------------------------------------------------ */

/* prologues: elementwise / normalisation work run inside the quantiser on the row it holds */
#define B200W4A4_PRE_NONE 0
#define B200W4A4_PRE_GELU_TANH 1      /* v = fp16(gelu_tanh(x)) */
#define B200W4A4_PRE_LAYERNORM_MOD 2  /* v = fp16(fp16(layernorm(x)) * (1 + scale[k]) + shift[k]) */
/* epilogues: elementwise work run inside the GEMM on y = fp16(acc*sa*sw + bias) */
#define B200W4A4_EPI_NONE 0
#define B200W4A4_EPI_GELU_TANH 1      /* out = fp16(gelu_tanh(y)) */
#define B200W4A4_EPI_GATE_RESIDUAL 2  /* out = fp16(float(residual) + float(y) * gate[n]) */

/* Quantiser with a fused prologue; x is fp16 [M,K], K <= 16384, codes go to the int8 container.
 * LAYERNORM_MOD folds the block-entry modulation of the DiT block,
 * `norm(x) * (1 + scale) + shift` (vdm_infer/models/wan_vdm/modules/dit_block.py:103, :113;
 * layer norm without affine evaluated in fp32 and cast to fp16 as diffusers' FP32LayerNorm does),
 * GELU_TANH the activation between the FFN projections (FeedForward "gelu-approximate",
 * dit_block.py:53, :114), into the per-token quantisation that follows them, so the
 * normalised / activated tensor is never written.  mod_scale / mod_shift are fp32 [K]
 * (mod_row_stride = 0) or one vector per token (mod_row_stride = K). */
int b200w4a4_quantize_act_fused(const void* x_f16, int prologue, const float* mod_scale,
                                const float* mod_shift, long long mod_row_stride, float ln_eps,
                                void* qact, float* act_scale, int M, int K, float clip,
                                void* stream);

/* GEMM with a fused epilogue.  GATE_RESIDUAL folds `hidden + out * gate`
 * (dit_block.py:105, :115; gate fp32 [N], or per token with gate_row_stride = N; residual fp16
 * [M,N], may be the same buffer as out), GELU_TANH the FFN activation. */
int b200w4a4_gemm_fused(const void* qact, const float* act_scale, const void* w_b200,
                        const void* w_scale, const void* bias, void* out, int epilogue,
                        const void* residual_f16, const float* gate, long long gate_row_stride, int M,
                        int N, int K, void* stream);

/* GEMM whose output columns go to `segments` (1..3) separate matrices: segment s holds columns
 * [s*N/segments, (s+1)*N/segments) as a [M, N/segments] fp16 matrix at outs[s] with a row pitch
 * of out_ld[s] elements (>= N/segments, a multiple of 8; base 16-byte aligned).  N/segments must
 * be a multiple of 64.  This is the fused QKV / KV projection writing q, k and v as contiguous
 * tensors - or straight into rows of a larger buffer, e.g. the slot of this rank in an
 * all-gather buffer - where the reference returns strided views of one [M,3D] matrix
 * (linear_vdm_w4a4_qkv, vdm_w4a4.py:297-298).  Values are those of b200w4a4_gemm. */
int b200w4a4_gemm_split(const void* qact, const float* act_scale, const void* w_b200,
                        const void* w_scale, const void* bias, void* const* outs,
                        const long long* out_ld, int segments, int M, int N, int K, void* stream);

/* b200w4a4_quantize_act_fused + b200w4a4_gemm_fused with the workspace of b200w4a4_linear. */
int b200w4a4_linear_fused(const void* x_f16, int prologue, const float* mod_scale,
                          const float* mod_shift, long long mod_row_stride, float ln_eps,
                          const void* w_b200, const void* w_scale, const void* bias, void* out,
                          int epilogue, const void* residual_f16, const float* gate,
                          long long gate_row_stride, void* workspace, size_t workspace_bytes, int M,
                          int N, int K, float clip, void* stream);

/* Per-token work between the fused QKV projection and the attention kernel, in one pass over
 * a [L,D] fp16 matrix (row pitch x_ld elements): RMSNorm across the whole row with an fp16
 * weight (norm_q / norm_k, vdm_infer/models/wan_vdm/modules/attention.py:167-168, :208-216),
 * rotary embedding on consecutive pairs inside each head (apply_rotary_emb, :131-135) and the
 * cast to the attention dtype.  norm_weight_f16 NULL skips the norm; rope_cos_sin NULL skips
 * the rotation (both NULL: a plain cast/copy).  rope_cos_sin is fp32 [L, head_dim/2, 2] =
 * (cos, sin) per token and pair, shared by all heads.  out is fp16 or bf16 (B200W4A4_F16 /
 * B200W4A4_BF16) [L,D] with row pitch out_ld.  D % 8 == 0, D <= 16384, head_dim % 8 == 0,
 * pitches multiples of 8.  Intermediate roundings are those of the reference ops
 * (fp16 after the normalisation, after the weight multiply and after the rotation). */
int b200w4a4_qk_norm_rope(const void* x_f16, long long x_ld, const void* norm_weight_f16,
                          const float* rope_cos_sin, float eps, int head_dim, void* out, int out_dtype,
                          long long out_ld, int L, int D, void* stream);

/* b200w4a4_qk_norm_rope whose result goes to n_outs (1..8) destination matrices at row offset
 * out_row0 - e.g. this rank's rows of the gathered K (or V) buffer of every GPU of a row-sharded
 * attention group, the peers' buffers being peer-mapped memory: plain stores, the all-gather
 * happens inside the producing kernel.  All destinations share dtype and row pitch.
 * flags / ticket (both or neither): when every store of the launch is visible system-wide, the
 * kernel writes `epoch` to flags[d][flag_index] for each destination d with a non-NULL flags[d]
 * (release, system scope).  flags[d] points into the memory of the GPU that owns destination d;
 * ticket is a zero-initialised unsigned int in this GPU's memory, zero again when the kernel ends.
 * The consumer calls b200w4a4_wait_flags on its own flag array before it reads the buffer. */
int b200w4a4_qk_norm_rope_push(const void* x_f16, long long x_ld, const void* norm_weight_f16,
                               const float* rope_cos_sin, float eps, int head_dim, void* const* outs,
                               int n_outs, int out_dtype, long long out_ld, long long out_row0,
                               uint32_t* const* flags, int flag_index, uint32_t epoch,
                               unsigned int* ticket, int L, int D, void* stream);

/* Merge of two partial attention results over disjoint key sets:
 *   out = o1 * w1 + o2 * w2,  w_i = exp(lse_i - logaddexp(lse1, lse2))
 * o1 / o2: bf16 [L, H*head_dim] with row pitches o1_ld / o2_ld (elements), lse1 / lse2: fp32 [H, L]
 * (log-sum-exp of the scaled scores, as attention kernels report it), out: bf16 [L, H*head_dim].
 * Lets a row-sharded rank attend to its own keys while its peers' keys are still arriving and
 * fold the two results afterwards.  No counterpart in the reference (its sequence-parallel
 * hooks are identity stubs, vdm_infer/models/wan_vdm/modules/attention.py:20-32). */
int b200w4a4_attn_merge(const void* o1_bf16, long long o1_ld, const void* o2_bf16, long long o2_ld,
                        const float* lse1, const float* lse2, void* out_bf16, int L, int H, int head_dim,
                        void* stream);

/* Enqueues a one-warp kernel that waits until flags[i] has reached `epoch` (wrap-around safe
 * comparison) for every i < n (n <= 32), for at most timeout_ms (1..10000).  A wait that runs out
 * records code 105 in the device status word (b200w4a4_last_device_status) and ends the kernel;
 * nothing traps and the context stays usable. */
int b200w4a4_wait_flags(const uint32_t* flags, int n, uint32_t epoch, int timeout_ms, void* stream);

/* Enqueues a kernel that writes `value` to flags[d][index] for d < n (n <= 8; NULL entries are
 * skipped) with release semantics at system scope, ordered after all earlier work of the stream:
 * the consumer's "done reading" signal that lets producers overwrite a gather buffer. */
int b200w4a4_signal_flags(uint32_t* const* flags, int n, int index, uint32_t value, void* stream);

/* Same result as b200w4a4_linear, for callers that cannot allocate device memory.
 * (No counterpart in the reference, whose ops allocate their intermediates with
 * torch::empty on every call.)
 *
 * Some hosts of this library may not call cudaMalloc or any allocator at the point where
 * they run a layer: code running inside a memory-pool or arena that was sized up front, a
 * real-time or serving loop that forbids allocator calls after start-up, an embedding
 * runtime that hands out device memory itself and has none to spare for a workspace.
 * b200w4a4_linear needs a caller-provided workspace for the quantised activations; this
 * entry point keeps that intermediate in an array that is part of the library image instead
 * (8 MiB of codes + 32 KiB of scales; every GPU that loads the library holds it until the
 * process exits).  The caller still passes x, the repacked weight, scales, bias and out.
 *
 * Limits: M <= b200w4a4_linear_noalloc_max_rows() (8192) and
 * M * K <= b200w4a4_linear_noalloc_max_codes() (8 Mi, e.g. 512 x 13824 or 1638 x 5120);
 * larger shapes return B200W4A4_ELIMIT and launch nothing.
 * It calls no cudaMalloc / cudaFree or other allocating routine.  The first call on a device
 * looks up the array's address on that device (and does this library's usual one-time
 * per-device set-up); make that first call before any stream capture begins.
 * All calls share the one array, which keeps whatever the last call left in it: two calls
 * that overlap on the GPU (different streams, or the same stream from two threads without
 * ordering) race on it.  Calls on one stream are ordered and safe. */
int b200w4a4_linear_noalloc(const void* x, int x_dtype, const void* w_b200, const void* w_scale,
                            const void* bias, void* out, int M, int N, int K, float clip,
                            void* stream);
size_t b200w4a4_linear_noalloc_max_codes(void);
int b200w4a4_linear_noalloc_max_rows(void);

/* ---- helpers ------------------------------------------------------------ */

/* Extract int8 codes [rows,K] from a packed buffer (parity tests). */
int b200w4a4_unpack_codes(const void* packed, int8_t* codes, int rows, int K, int which,
                          void* stream);

/* Select the GEMM variant: 1 = one CTA per 128x256 tile, 2 = CTA pair per
 * 256x256 tile (cta_group::2).  Returns the previous value, or EINVAL. */
int b200w4a4_set_cta_group(int cta_group);

/* Select how the GEMM stages the weight operand; returns the previous value, or EINVAL
 * (0 only asks for the current value).
 *   4 (default)  the weight stays packed int4 in HBM and L2; TMA stages packed tiles and warps
 *                of the GEMM widen them to int8 in shared memory (tcgen05 has no s4 kind);
 *   8            b200w4a4_repack_weight writes int8 [N,K] (every byte 16 * code) and TMA stages it
 *                straight into the tile the tensor core reads: no widening work inside the GEMM
 *                (measured +5 % on the Wan-14B shapes, +10 % at K = 1536) for twice the weight bytes.
 * The choice is process-wide and decides the meaning of every `w_b200` pointer and the size
 * b200w4a4_repack_bytes returns: make it before any weight is repacked.  The environment variable
 * B200W4A4_WEIGHT_STAGING=int8 selects 8 at first use.  No counterpart in the reference, whose
 * kernel feeds s4 operands to mma.sync directly (vdm_w4a4_kernel.cu:114-143). */
int b200w4a4_set_weight_staging(int bits);

/* Synchronises `device`, returns and clears its device status word:
 * 0, or the code (> 0) of the kernel role whose bounded wait ran out
 * (101-104: a role of the GEMM; 105: b200w4a4_wait_flags).  The word is a report
 * only: it keeps the first code until it is read here and never cancels a later
 * launch (a GEMM gives up early only on a time-out of its own launch).
 * No counterpart in the reference, whose kernels have no waits to bound. */
int b200w4a4_last_device_status(int device);

/* Synchronises `device` and returns B200W4A4_OK, or B200W4A4_EDEVICE when a kernel
 * has recorded a time-out since the word was last cleared (the word is left as it
 * is, so b200w4a4_last_device_status still tells which role).  The reference
 * surfaces device-side failures through TORCH_CHECK / cudaGetLastError after its
 * launches (vdm_w4a4_kernel.cu:700-728, 765-838); this is the explicit form. */
int b200w4a4_check_device(int device);

/* Tensor-map table statistics: launches whose TMA descriptors were found in the
 * library's table (hits) or had to be encoded by the driver (misses).  Either
 * pointer may be NULL.  No counterpart in the reference (it uses no TMA). */
void b200w4a4_map_cache_stats(unsigned long long* hits, unsigned long long* misses);

#ifdef __cplusplus
}
#endif
#endif /* B200W4A4_H_ */
