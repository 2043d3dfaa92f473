/*
 * quamba_b200 -- C ABI of the B200 (sm_100a) quantized Mamba mixer kernels.
 *
 * Every entry point takes a pointer to a plain-old-data argument struct and the CUDA
 * stream to enqueue on (a cudaStream_t passed as void*), returns a qb_status, never
 * synchronises the host, never allocates device memory, and borrows every buffer.
 * Device pointers are raw addresses on the current device; strides are in ELEMENTS.
 * Scales that the reference passes as CUDA tensors stay device pointers (const float*);
 * scales that the reference passes as Python floats are floats by value.
 *
 * The struct definitions below are also parsed by the Python loader (one field per
 * line, "type name;"), so keep that shape when editing.
 *
 * "Replaces" comments cite the reference interface (path inside the reference project).
 */
#ifndef QUAMBA_B200_H_
#define QUAMBA_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum {
  QB_OK = 0,
  QB_ERR_INVALID_ARG = -1, /* shape / stride / alignment / null pointer rejected on the host */
  QB_ERR_UNSUPPORTED = -2, /* a configuration the reference also rejects, or not built yet  */
  QB_ERR_CUDA = -3,        /* a CUDA runtime call or launch failed                          */
  QB_ERR_TIMEOUT = -4,     /* a bounded device-side wait expired (read from a status word)  */
  QB_ERR_TOO_LARGE = -5    /* a size beyond a stated maximum                                */
} qb_status;

/* Human-readable text of the last non-OK status returned on the calling thread. */
const char* qb_last_error(void);
/* Library ABI version (bumped when a struct changes). */
int qb_abi_version(void);
/* sizeof() of an argument struct by name, for binding self-checks; -1 if unknown. */
int64_t qb_sizeof(const char* struct_name);
/* Cross-check switches: a bit set here sends the op to its portable twin (the five-stage SSD path, the SIMT Hadamard
 * kernel, the 128 x 128 GEMM kernel, the CTA-tile state update) so that two implementations can be compared on one
 * device.  Process-wide, off by default, never read from the environment.  Returns the previous mask. */
#define QB_PATH_SSD_PORTABLE 1
#define QB_PATH_HADAMARD_SIMT 2
#define QB_PATH_GEMM_SMALL_TILES 4
#define QB_PATH_UPDATE_CTA_TILES 8
int qb_set_path_override(int mask);
/* Caps the number of multiprocessors the library's kernels size their grids for (persistent kernels launch one CTA per
 * SM of the budget; one-wave grids are cut for it).  0 (default) = all SMs of the device.  A caller that overlaps these
 * kernels with a collective on another stream leaves the collective's CTAs room this way: a persistent grid that fills
 * every SM lets the collective start only when a kernel ends, and a collective that got in first makes the next
 * persistent grid run in two waves.  Results do not depend on the budget.  Process-wide; returns the previous value.
 * No reference counterpart. */
int qb_set_sm_budget(int sms);
/* While on (non-zero), the kernels of a prefill chain -- norms, the tensor-core GEMMs, conv1d forward, the SSD scan, the
 * Hadamard kernel -- signal as they start that the NEXT programmatic launch on the stream may become resident and run its
 * prologue (barrier and tensor-memory set-up, constant tables, weight prefetch) while they still work; its
 * griddepcontrol.wait then holds it until this kernel's results are complete.  What follows such a kernel on the stream
 * must be a kernel of this library (all of them read activations through L2, by TMA / bulk copies or ld.global.cg, which an
 * early start requires) or an ordinary launch (which waits for full completion anyway).  Off by default; the model's
 * forward switches it on around its own launch sequence.  Process-wide; returns the previous value.  No reference
 * counterpart. */
int qb_set_early_overlap(int on);
/* Synchronises `stream`, then returns and clears the device status word: QB_OK, or QB_ERR_TIMEOUT
 * if a kernel gave up on a bounded wait (its outputs are then undefined).  The only entry point
 * that blocks the host. */
int qb_read_device_status(void* stream);

/* ------------------------------------------------------------------------------------------
 * int8 causal conv1d, Quamba1 (one scale set for all channels).
 * Replaces quant_causal_conv1d_cuda.fwd / .update
 *   (csrc/causal_conv1d/quant_causal_conv1d.cpp:77-164, :168-226).
 * y = silu( scale_w*scale_x * sum_w w[c,w] x[c, l-(W-1-w)] + scale_b*bias[c] ),
 * q_y = clamp(roundf(y / scale_out)).  x (B, D, L) with either L or D contiguous
 * (x_sl == 1 or x_sd == 1); out has the same strides as x.  width 2..4.
 * ------------------------------------------------------------------------------------------ */
typedef struct {
  const int8_t* x;
  int8_t* out;
  const int8_t* weight;
  const int8_t* bias;
  int64_t x_sb;
  int64_t x_sd;
  int64_t x_sl;
  int64_t out_sb;
  int64_t out_sd;
  int64_t out_sl;
  int32_t batch;
  int32_t dim;
  int32_t seqlen;
  int32_t width;
  float scale_x;
  float scale_w;
  float scale_out;
  float scale_b;
  int32_t silu;
} qb_conv1d_fwd_args;
int qb_causal_conv1d_fwd(const qb_conv1d_fwd_args* a, void* stream);

/* Decode step: conv_state (B, D, W) int8 (any strides) is shifted left by one and x appended,
 * in place; out (B, D) int8. */
typedef struct {
  const int8_t* x;
  int8_t* conv_state;
  int8_t* out;
  const int8_t* weight;
  const int8_t* bias;
  int64_t x_sb;
  int64_t x_sd;
  int64_t state_sb;
  int64_t state_sd;
  int64_t state_sw;
  int64_t out_sb;
  int64_t out_sd;
  int32_t batch;
  int32_t dim;
  int32_t width;
  float scale_x;
  float scale_w;
  float scale_out;
  float scale_b;
  int32_t silu;
} qb_conv1d_update_args;
int qb_causal_conv1d_update(const qb_conv1d_update_args* a, void* stream);

/* ------------------------------------------------------------------------------------------
 * int8 causal conv1d, Quamba2: one pass over the concatenated [x | B | C] channels with
 * per-segment input / weight / bias scales, per-(ssd group, head group, dim group) output
 * scales for x and per-ssd-group output scales for B and C; writes three tensors.
 * Replaces quamba2_conv1d_cuda.fwd / .update
 *   (csrc/causal_conv1d/quamba2_conv1d.cpp:122-260, :263-380).
 * xBC (B, dim, L) channel-last: element (b, c, l) at b*xBC_sb + l*xBC_sl + c.
 * Outputs x (B, L, x_dim), Bm / Cm (B, L, d_state*n_groups), all contiguous.
 * head_group_range / dim_group_range null  =>  x_scales, B_scales, C_scales have 1 element.
 * ------------------------------------------------------------------------------------------ */
typedef struct {
  const int8_t* xBC;
  int8_t* x;
  int8_t* Bm;
  int8_t* Cm;
  const int8_t* weight;
  const int8_t* bias;
  const int32_t* head_group_range;
  const int32_t* dim_group_range;
  const float* x_scales;
  const float* B_scales;
  const float* C_scales;
  int64_t xBC_sb;
  int64_t xBC_sl;
  int32_t batch;
  int32_t dim;
  int32_t seqlen;
  int32_t width;
  int32_t x_dim;
  int32_t x_headdim;
  int32_t d_state;
  int32_t n_groups;
  int32_t nhead_groups;
  int32_t ndim_groups;
  float scale_x;
  float scale_B;
  float scale_C;
  float scale_wx;
  float scale_wB;
  float scale_wC;
  float scale_bx;
  float scale_bB;
  float scale_bC;
  int32_t silu;
} qb_quamba2_conv1d_fwd_args;
int qb_quamba2_conv1d_fwd(const qb_quamba2_conv1d_fwd_args* a, void* stream);

/* Decode step: xBC (B, dim); conv_state element (b, c, w) at b*state_sb + c*state_sd + w*state_sw,
 * updated in place; outputs x (B, x_dim), Bm / Cm (B, d_state*n_groups) contiguous. */
typedef struct {
  const int8_t* xBC;
  int8_t* conv_state;
  int8_t* x;
  int8_t* Bm;
  int8_t* Cm;
  const int8_t* weight;
  const int8_t* bias;
  const int32_t* head_group_range;
  const int32_t* dim_group_range;
  const float* x_scales;
  const float* B_scales;
  const float* C_scales;
  int64_t xBC_sb;
  int64_t state_sb;
  int64_t state_sd;
  int64_t state_sw;
  int32_t batch;
  int32_t dim;
  int32_t width;
  int32_t x_dim;
  int32_t x_headdim;
  int32_t d_state;
  int32_t n_groups;
  int32_t nhead_groups;
  int32_t ndim_groups;
  float scale_x;
  float scale_B;
  float scale_C;
  float scale_wx;
  float scale_wB;
  float scale_wC;
  float scale_bx;
  float scale_bB;
  float scale_bC;
  int32_t silu;
} qb_quamba2_conv1d_update_args;
int qb_quamba2_conv1d_update(const qb_quamba2_conv1d_update_args* a, void* stream);

/* ------------------------------------------------------------------------------------------
 * Fused Hadamard rotation + int8 quantisation: out = sat_int8(roundf((H_dim x) * scale)).
 * Replaces quant_hadamard.fast_hadamard_transform{,_12N,_20N,_28N,_40N}
 *   (csrc/hadamard/quant_hadamard.cpp:72-294).
 * x (rows, dim) row-contiguous, in_dtype 0 = fp16, 1 = bf16, 2 = fp32.  special = 1 (dim a power
 * of two) or 12 / 20 / 28 / 40 (dim = special * 2^k).  Unlike the reference (which casts an
 * out-of-range float to int8, undefined), the result saturates to [-128, 127].
 * ------------------------------------------------------------------------------------------ */
typedef struct {
  const void* x;
  int8_t* out;
  int64_t x_row_stride;
  int64_t out_row_stride;
  int64_t rows;
  int32_t dim;
  int32_t special;
  int32_t in_dtype;
  float scale;
} qb_hadamard_quant_args;
int qb_hadamard_quant(const qb_hadamard_quant_args* a, void* stream);

/* ------------------------------------------------------------------------------------------
 * Mamba1 int8 selective scan forward.
 * Replaces quant_sscan_cuda.fwd (csrc/selective_scan/quant_sscan.cpp:122-265).
 * u, delta, z: (B, D, L) int8, L contiguous.  Bm, Cm: (B, G, N, L) int8, L contiguous.
 * A_log (D, N) int8, D / delta_bias (D) int8 (nullable).  out: (B, L, D) fp16 contiguous (the
 * transposed layout the reference returns).  x_states: (B, D, nchunks, N) int8, nchunks =
 * ceil(L / 2048): the state after each 2048-step chunk, quantised with roundf + clamp.
 * All *_scale are device pointers to one float.
 * ------------------------------------------------------------------------------------------ */
typedef struct {
  const int8_t* u;
  const int8_t* delta;
  const int8_t* z;
  const int8_t* Bm;
  const int8_t* Cm;
  const int8_t* A_log;
  const int8_t* D;
  const int8_t* delta_bias;
  const float* u_scale;
  const float* delta_scale;
  const float* z_scale;
  const float* B_scale;
  const float* C_scale;
  const float* A_scale;
  const float* D_scale;
  const float* delta_bias_scale;
  const float* ssm_state_scale;
  void* out;
  int8_t* x_states;
  int64_t u_sb;
  int64_t u_sd;
  int64_t delta_sb;
  int64_t delta_sd;
  int64_t z_sb;
  int64_t z_sd;
  int64_t B_sb;
  int64_t B_sg;
  int64_t B_sn;
  int64_t C_sb;
  int64_t C_sg;
  int64_t C_sn;
  int32_t batch;
  int32_t dim;
  int32_t seqlen;
  int32_t dstate;
  int32_t n_groups;
  int32_t delta_softplus;
} qb_sscan_fwd_args;
int qb_sscan_fwd(const qb_sscan_fwd_args* a, void* stream);

/* ------------------------------------------------------------------------------------------
 * Single-step state update (decode), int8 state updated in place.
 * Replaces quant_sscan_update_triton / quamba2_sscan_update_triton
 *   (quamba/triton/selective_state_update.py:129-227, :365-478).
 * state (B, H, P, N) int8 contiguous in N (Mamba1: H = 1, P = d_inner).  x (B, H, P) int8;
 * dt int8 with strides (dt_sb, dt_sh, dt_sp) (dt_sp = 0 when tied across P); A_log int8 with
 * strides (A_sh, A_sp, A_sn) (0 strides when tied); Bm / Cm (B, G, N) int8; D int8 strides
 * (D_sh, D_sp), nullable; z like x, nullable.  dt_bias: int8 + dt_bias_scale (Mamba1), or fp16
 * added unscaled when dt_bias_is_half != 0 (Mamba2); strides (bias_sh, bias_sp).
 * Scale layouts: per-tensor (grouped == 0: x_scales / state_scale / B_scale / C_scale point to
 * one float) or grouped (x_scales [G,HG,DG], state_scale [G,HG,DG,N], B_scale / C_scale [G],
 * ranges as in the conv).  State requantised with rint (half to even) + clamp; out (B, H, P)
 * fp16 uses the un-requantised fp32 state.  early_launch: see the decode entry points below; 0 unless the next kernel
 * on the stream is one of them.
 * ------------------------------------------------------------------------------------------ */
typedef struct {
  int8_t* state;
  const int8_t* x;
  const int8_t* dt;
  const int8_t* A_log;
  const int8_t* Bm;
  const int8_t* Cm;
  const int8_t* D;
  const int8_t* z;
  const void* dt_bias;
  const float* x_scales;
  const float* dt_scale;
  const float* A_scale;
  const float* state_scale;
  const float* B_scale;
  const float* C_scale;
  const float* D_scale;
  const float* z_scale;
  const float* dt_bias_scale;
  const int32_t* head_group_range;
  const int32_t* dim_group_range;
  void* out;
  int64_t state_sb;
  int64_t state_sh;
  int64_t state_sp;
  int64_t x_sb;
  int64_t x_sh;
  int64_t dt_sb;
  int64_t dt_sh;
  int64_t dt_sp;
  int64_t A_sh;
  int64_t A_sp;
  int64_t A_sn;
  int64_t B_sb;
  int64_t B_sg;
  int64_t C_sb;
  int64_t C_sg;
  int64_t D_sh;
  int64_t D_sp;
  int64_t z_sb;
  int64_t z_sh;
  int64_t bias_sh;
  int64_t bias_sp;
  int64_t out_sb;
  int64_t out_sh;
  int32_t batch;
  int32_t nheads;
  int32_t headdim;
  int32_t dstate;
  int32_t ngroups;
  int32_t grouped;
  int32_t nhead_groups;
  int32_t ndim_groups;
  int32_t dt_bias_is_half;
  int32_t dt_softplus;
  int32_t early_launch;
} qb_sscan_update_args;
int qb_sscan_update(const qb_sscan_update_args* a, void* stream);

/* ------------------------------------------------------------------------------------------
 * Mamba2 int8 SSD chunk scan with inter-chunk state passing.
 * Replaces _quant_mamba_chunk_scan_combined_fwd / _quamba2_mamba_chunk_scan_combined_fwd
 *   (quamba/triton/quant_ssd_combined.py:11-81, :84-166) and the six Triton kernels below them.
 * x (B, L, H, P) int8, P contiguous, strides (x_sb, x_sl, x_sh); dt (B, L, H) int8 with strides
 * (dt_sb, dt_sl), H contiguous; Bm / Cm (B, L, G, N) int8, N contiguous, strides (sb, sl, sg);
 * A_log (H) int8; D (H) or (H, P) int8, nullable; dt_bias (H) fp16, nullable; z like x, nullable.
 * out (B, L, H, P) fp16 contiguous; final_states (B, H, P, N) int8 contiguous (rint + clamp).
 * Scales: grouped == 0 => x_scales / ssm_state_scale / B_scale / C_scale point to one float;
 * grouped != 0 => [G,HG,DG], [G,HG,DG,N], [G], [G] with the cumulative range tables.
 * workspace: device scratch of at least qb_ssd_workspace_bytes() bytes, 256-byte aligned;
 * contents are undefined on entry and on exit.
 * ------------------------------------------------------------------------------------------ */
typedef struct {
  const int8_t* x;
  const int8_t* dt;
  const int8_t* Bm;
  const int8_t* Cm;
  const int8_t* A_log;
  const int8_t* D;
  const int8_t* z;
  const void* dt_bias;
  const float* x_scales;
  const float* dt_scale;
  const float* A_scale;
  const float* B_scale;
  const float* C_scale;
  const float* D_scale;
  const float* z_scale;
  const float* ssm_state_scale;
  const int32_t* head_group_range;
  const int32_t* dim_group_range;
  void* out;
  int8_t* final_states;
  void* workspace;
  int64_t workspace_bytes;
  int64_t x_sb;
  int64_t x_sl;
  int64_t x_sh;
  int64_t dt_sb;
  int64_t dt_sl;
  int64_t B_sb;
  int64_t B_sl;
  int64_t B_sg;
  int64_t C_sb;
  int64_t C_sl;
  int64_t C_sg;
  int64_t z_sb;
  int64_t z_sl;
  int64_t z_sh;
  int32_t batch;
  int32_t seqlen;
  int32_t nheads;
  int32_t headdim;
  int32_t ngroups;
  int32_t dstate;
  int32_t chunk_size;
  int32_t grouped;
  int32_t nhead_groups;
  int32_t ndim_groups;
  int32_t D_has_hdim;
  int32_t dt_softplus;
  float dt_min;
  float dt_max;
} qb_ssd_args;
int64_t qb_ssd_workspace_bytes(int32_t batch, int32_t seqlen, int32_t nheads, int32_t headdim,
                               int32_t ngroups, int32_t dstate, int32_t chunk_size);
int qb_ssd_chunk_scan_fwd(const qb_ssd_args* a, void* stream);

/* The same SSD forward for callers that cannot provide scratch memory.  (No counterpart in the
 * reference, whose Triton wrappers allocate their intermediates through torch.)  A host program
 * without a device allocator of its own, or one whose memory pool is sealed after model load, has
 * no way to obtain the workspace above short of cudaMalloc; this entry point therefore ignores
 * a->workspace / a->workspace_bytes and uses an array built into the library's device image
 * (qb_ssd_static_scratch_bytes() bytes, 48 MiB, resident on every GPU that loads the library until
 * the process exits).  It calls no cudaMalloc / cudaFree and no allocating library routine; inputs
 * and outputs are still the caller's.  Shapes whose workspace (qb_ssd_workspace_bytes) exceeds the
 * array are rejected with QB_ERR_TOO_LARGE.  The first call on each device looks up the array's
 * device address and should therefore be made before any stream capture begins.  All calls share the
 * one array: two calls whose kernels can overlap on the GPU (different streams) race on it; calls
 * on one stream are safe, and nothing needs clearing between them. */
int64_t qb_ssd_static_scratch_bytes(void);
int qb_ssd_chunk_scan_fwd_noalloc(const qb_ssd_args* a, void* stream);

/* ------------------------------------------------------------------------------------------
 * W4A8 linears (Marlin-QQQ packed int4 weights, int8 activations).
 * Replaces quant_linear_cuda.w4a8o16_gemm / w4a8o8_gemm
 *   (csrc/linear/marlin_qqq_gemm_kernel.cuh:1187-1314, marlin_qqq_gemm_kernel_o8.cuh:1199-).
 *
 * qb_w4a8_unpack converts the module's buffers (weight int32 (K/16, N*16/8) in the Marlin-QQQ
 * tile order, s_group fp16 (K/128, N) and s_channel fp32 (1, N) in their permuted orders) into
 * the layout the B200 kernels stream: w8 int8 (N, K) K-contiguous holding exactly the int8
 * values the reference multiplies with (per-group: (q-8)*s_group rounded half-to-even by one
 * fp16 fma; per-channel: 16*q), and s_channel_nat fp32 (N) in natural column order.  It is a
 * one-time (or per-call, it is cheap) preparation; s_group == null selects per-channel.
 *
 * qb_w4a8_gemm: acc = a (M,K) int8 @ w8^T, out = acc * s_channel[n] * s_tok -> fp16 (cvt.rn) or
 * int8 (cvt.rni, saturating); s_tok has 1 element or M elements (s_tok_per_row).  out is (M, N)
 * row-major, or (N, M) when output_transpose != 0.  out_row_stride in elements.
 * ------------------------------------------------------------------------------------------ */
typedef struct {
  const int32_t* packed;
  const void* s_group;
  const float* s_channel;
  int8_t* w8;
  float* s_channel_nat;
  int32_t size_k;
  int32_t size_n;
  int32_t group_size;
} qb_w4a8_unpack_args;
int qb_w4a8_unpack(const qb_w4a8_unpack_args* a, void* stream);

typedef struct {
  const int8_t* a;
  const int8_t* w8;
  const float* s_channel_nat;
  const float* s_tok;
  void* out;
  int64_t a_row_stride;
  int64_t out_row_stride;
  int32_t m;
  int32_t n;
  int32_t k;
  int32_t s_tok_per_row;
  int32_t out_int8;
  int32_t output_transpose;
} qb_w4a8_gemm_args;
int qb_w4a8_gemm(const qb_w4a8_gemm_args* a, void* stream);

/* Decode-sized W4A8 product (1 <= m < 32) straight from 4-bit weights, for per-channel quantised weights (no group
 * scales): the same result as qb_w4a8_gemm, bit for bit, from half the weight bytes.  (The reference has one kernel for
 * all m, marlin_qqq_gemm_kernel.cuh:1187-1314; this is the small-m case of the same call.)
 * qb_w4a8_pack_nibbles builds the weight copy it reads from the int8 copy qb_w4a8_unpack made: w4 (n, k / 2) bytes;
 * 32-bit word i of a row covers k = 8 i .. 8 i + 7, value + 8 of k = 8 i + b in the low and of k = 8 i + 4 + b in the high
 * nibble of byte b.  k must be a multiple of 32, a rows 16-byte aligned. */
typedef struct {
  const int8_t* a;
  const uint8_t* w4;
  const float* s_channel_nat;
  const float* s_tok;
  void* out;
  int64_t a_row_stride;
  int64_t out_row_stride;
  int32_t m;
  int32_t n;
  int32_t k;
  int32_t s_tok_per_row;
  int32_t out_int8;
  int32_t output_transpose;
} qb_w4a8_gemv_s4_args;
int qb_w4a8_pack_nibbles(const int8_t* w8, uint8_t* w4, int32_t n, int32_t k, void* stream);
int qb_w4a8_gemv_s4(const qb_w4a8_gemv_s4_args* a, void* stream);

/* ------------------------------------------------------------------------------------------
 * W8A8 linears.
 * Replaces quant_linear_cuda.cutlass_scaled_mm_dq / cutlass_scaled_mv_dq / w8a8o8_gemv
 *   (csrc/linear/quant_linear_fwd_kernel.cuh:356-401, quant_linear_fwd_gemv_kernel.cuh:96-134).
 * D (M, N) = cvt( a_scale (.) ( b_scale (.) float(A (M,K) @ B (K,N)) ) ) with A row-major
 * (a_row_stride) and B column-major (element (k, n) at n*b_col_stride + k); a_scale has 1 or M
 * elements, b_scale 1 or N.  out_dtype 0 = int8 (round half to even, saturating), 1 = fp16,
 * 2 = bf16.  The "mv" forms of the reference are this call with M = 1 and the scalars in
 * alpha (by value, use_alpha != 0) or roundf rounding (round_half_away != 0, w8a8o8_gemv).
 * ------------------------------------------------------------------------------------------ */
typedef struct {
  const int8_t* a;
  const int8_t* b;
  const float* a_scale;
  const float* b_scale;
  void* out;
  int64_t a_row_stride;
  int64_t b_col_stride;
  int64_t out_row_stride;
  int32_t m;
  int32_t n;
  int32_t k;
  int32_t a_scale_per_row;
  int32_t b_scale_per_col;
  int32_t out_dtype;
  int32_t use_alpha;
  int32_t round_half_away;
  float alpha;
} qb_w8a8_gemm_args;
int qb_w8a8_gemm(const qb_w8a8_gemm_args* a, void* stream);

/* Measurement aid (no counterpart in the reference): the dense int8 rate of tcgen05.mma kind::i8 on the current device,
 * operands resident in shared memory, one CTA per SM, `repeats` launches of `groups` x four M128 N256 K32 MMAs each, timed
 * with CUDA events.  *tops receives TOP/s (2 x MACs), *ms (nullable) the elapsed time.  Blocks the host.  The GEMM
 * rooflines use this figure as their peak. */
int qb_i8_mma_peak(int groups, int repeats, void* stream, double* tops, double* ms);

/* ------------------------------------------------------------------------------------------
 * Quantised RMSNorm with residual add, and gated grouped RMSNorm.
 * qb_rmsnorm_quant replaces _qlayer_norm_fwd (quamba/triton/quant_norm.py:68-206, called by
 *   QRMSNorm.forward, quamba/qNorm.py:52-87): h = x (+ residual); residual_out = h (stored in its
 *   own dtype); y = h * rstd * weight (+ bias), rstd = 1 / sqrt(mean(h^2) + eps) (is_rms_norm != 0;
 *   otherwise the mean is removed first); ngroups must be 1, z null.
 * qb_rmsnorm_gated replaces _qlayer_normgated_fwd (quamba/triton/quant_normgated.py:11-132, called
 *   by QRMSNormGated.forward, quamba/qNorm.py:145-174): each row is ngroups segments of group_size
 *   elements normalised on their own; z int8 (nullable) gates with g = z_scale*z, silu(g) = g*sigmoid(g):
 *   x*silu(g) before the norm (norm_before_gate == 0) or y*silu(g) after it; no residual.
 * x, weight, bias fp16; residual / residual_out fp16 or fp32 (the *_is_f32 flags).
 * out_kind 0: int8 = clamp(rint(y / out_scale));  1: int8 with one scale per (group, row),
 * scale = max(y) / 127 written to dyn_scale[group * rows + row] (the reference takes the maximum of y,
 * not of |y|, over a power-of-two block padded with zeros; reproduced);  2: fp16.
 * Row strides in elements.  group_size * 2 must stay below 64 KB as in the reference.
 * qb_rmsnorm_quant only, n_partials > 1 (no reference counterpart; the reduce half of a head-parallel layer's exchange
 * fused into the block norm): the input row is fp16(sum over p < n_partials of partial p), the sum taken in fp32 in the
 * order p = 0, 1, ...; partial p is x + p * partial_stride (elements), except p == own_index when own_partial != NULL,
 * which is read from own_partial (same row stride as x).  0 or 1: x alone.
 * ------------------------------------------------------------------------------------------ */
typedef struct {
  const void* x;
  const void* residual;
  void* residual_out;
  const int8_t* z;
  const void* weight;
  const void* bias;
  void* out;
  float* dyn_scale;
  int64_t x_row_stride;
  int64_t residual_row_stride;
  int64_t residual_out_row_stride;
  int64_t z_row_stride;
  int64_t out_row_stride;
  int32_t rows;
  int32_t group_size;
  int32_t ngroups;
  int32_t residual_is_f32;
  int32_t residual_out_is_f32;
  int32_t out_kind;
  int32_t norm_before_gate;
  int32_t is_rms_norm;
  float eps;
  float out_scale;
  float z_scale;
  int32_t n_partials;
  int32_t own_index;
  int64_t partial_stride;
  const void* own_partial;
} qb_rmsnorm_args;
int qb_rmsnorm_quant(const qb_rmsnorm_args* a, void* stream);
int qb_rmsnorm_gated(const qb_rmsnorm_args* a, void* stream);

/* ------------------------------------------------------------------------------------------
 * Token embedding gather with fp16 output.
 * Replaces quant_embedding_cuda.w4a16_embedding_lookup / w8a16_embedding_lookup
 *   (csrc/embedding/quant_embedding_kernel.cuh:47-139, :172-260) and torch's fp16 nn.Embedding.
 * kind 0: table fp16 (vocab, dim).  kind 1: table int8 (vocab, dim), scales fp16 (vocab):
 * out = scale * half(q).  kind 2: table int32 (vocab, dim / 8), eight 4-bit values (+8) per word
 * with nibble i holding element [0,2,4,6,1,3,5,7][i], scales fp16 (vocab): out = half(q - 8) * scale.
 * tokens int64 (n_tokens); out fp16 (n_tokens, dim) contiguous.  A token id outside [0, vocab)
 * reads row 0 and is reported by qb_read_device_status.
 * ------------------------------------------------------------------------------------------ */
typedef struct {
  const void* table;
  const void* scales;
  const int64_t* tokens;
  void* out;
  int64_t n_tokens;
  int32_t dim;
  int32_t vocab;
  int32_t kind;
} qb_embedding_args;
int qb_embedding_lookup(const qb_embedding_args* a, void* stream);

/* Greedy next token: out[r] = index of the largest of the n fp16 logits of row r (lowest index among equals).
 * Replaces the logits.argmax(dim=-1) of the reference's greedy decode loop (profile_mamba.py:317-392), so that a
 * captured decode step can feed its own next input.  row_stride in elements; at most 1024 rows per call.  The kernel
 * keeps its partial results in a small array inside the library: calls that can overlap on the GPU (different streams)
 * must not be issued concurrently. */
int qb_argmax_rows(const void* logits, int64_t row_stride, int32_t rows, int32_t n, int64_t* out, void* stream);

/* ------------------------------------------------------------------------------------------
 * Fused decode-step kernels for 1 to 4 rows (one token per sequence).  The reference launches these ops one by one
 * (block QRMSNorm, quamba/qNorm.py:52-87, then W4A8QMamba2.step, quamba/qMamba2.py:997-1020); here four launches cover
 * a layer (these two, the state update and the out_proj product), each bit-compatible with the separate entry points above up to their stated tolerances.
 *
 * early_launch (here, in qb_decode_gate_had_quant_args and in qb_sscan_update_args): non-zero lets the NEXT kernel on the
 *   stream start its own set-up while this one still runs (programmatic dependent launch).  Set it only when that next
 *   kernel is one of these decode entry points (or qb_sscan_update on its one-CTA-per-head path, or qb_argmax_rows): they read
 *   their producer's output past the L1 cache, which an early start requires; other kernels of the library do not.
 * qb_decode_norm_linear: h = x (+ residual); residual_out = h; a = int8(rmsnorm(h) * norm_weight / norm_out_scale);
 *   out (rows, n) = a @ W^T scaled by s_channel_nat[n] * s_tok, int8 (rint, saturating) or fp16.  W is the int8 copy
 *   qb_w4a8_unpack makes (n, k), or with w_is_s4 != 0 the nibble copy qb_w4a8_pack_nibbles makes (per-channel weights).
 *   With w_is_s4 != 0 and s_group_nat != null the weight is a GROUP-128 one streamed as 4 bits: w holds the raw codes in
 *   the same nibble layout (byte b of 32-bit word i of a row: code of k = 8 i + b low, of k = 8 i + 4 + b high) and
 *   s_group_nat the fp16 group scales in natural order, (n, k / 128) row-major; the kernel rebuilds the int8 weights
 *   (q - 8) * s_group in registers with the reference's own fp16 fma (marlin_qqq_gemm_kernel.cuh:136-178), so the result
 *   equals the product with the int8 copy bit for bit from half the bytes.
 *   With a_int8 != null (rows x k int8, row stride x_row_stride) the norm is skipped and a_int8 is multiplied as it is:
 *   the plain decode-sized product with this kernel's load scheduling.
 *   With conv_state != null the columns [conv_col0, conv_col0 + conv_dim) are not stored: each is fed to that channel's
 *   quamba2_conv1d update (width 4, per-tensor output scales; state element (b, c, w) at b*sb + c*sd + w*sw shifted in
 *   place) and the conv results go to conv_x (rows, conv_x_dim), conv_B / conv_C (rows, conv_gn).
 *   conv_scale_in_* = weight scale * input scale of the segment; conv_scale_bias_* = bias scale.
 * qb_decode_gate_had_quant: g = y * silu(z_scale * z); grouped rmsnorm(g) * norm_weight rounded to fp16; Hadamard
 *   rotation of length d (d / 128 in {12, 20, 28, 40} or a power of two <= 64; the norm group size a multiple of 128);
 *   out (rows, d) int8 = sat(roundf(. * had_scale)): QRMSNormGated + QHadamard (quamba/qNorm.py:145-174,
 *   quamba/qHadamard.py:31-35) in one launch, for any number of rows.
 * ------------------------------------------------------------------------------------------ */
typedef struct {
  const void* x;
  const int8_t* a_int8;
  const void* residual;
  void* residual_out;
  const void* norm_weight;
  const void* w;
  const float* s_channel_nat;
  const void* s_group_nat;
  const float* s_tok;
  void* out;
  int8_t* conv_state;
  const int8_t* conv_weight;
  const int8_t* conv_bias;
  int8_t* conv_x;
  int8_t* conv_B;
  int8_t* conv_C;
  const float* x_out_scale;
  const float* B_out_scale;
  const float* C_out_scale;
  int64_t x_row_stride;
  int64_t residual_row_stride;
  int64_t residual_out_row_stride;
  int64_t out_row_stride;
  int64_t conv_state_sb;
  int64_t conv_state_sd;
  int64_t conv_state_sw;
  int32_t rows;
  int32_t n;
  int32_t k;
  int32_t w_is_s4;
  int32_t out_int8;
  int32_t residual_is_f32;
  int32_t residual_out_is_f32;
  int32_t conv_col0;
  int32_t conv_dim;
  int32_t conv_x_dim;
  int32_t conv_gn;
  int32_t early_launch;
  float eps;
  float norm_out_scale;
  float conv_scale_in_x;
  float conv_scale_in_B;
  float conv_scale_in_C;
  float conv_scale_bias_x;
  float conv_scale_bias_B;
  float conv_scale_bias_C;
} qb_decode_norm_linear_args;
int qb_decode_norm_linear(const qb_decode_norm_linear_args* a, void* stream);

typedef struct {
  const void* y;
  const int8_t* z;
  const void* norm_weight;
  int8_t* out;
  int64_t y_row_stride;
  int64_t z_row_stride;
  int64_t out_row_stride;
  int32_t rows;
  int32_t d;
  int32_t group_size;
  int32_t early_launch;
  float z_scale;
  float eps;
  float had_scale;
} qb_decode_gate_had_quant_args;
int qb_decode_gate_had_quant(const qb_decode_gate_had_quant_args* a, void* stream);

/* ---- the exchange step of a head-parallel layer over peer memory ------------------------------------------------------
 * The reference has no tensor parallelism (quamba/qMamba2.py:84-88 asserts process_group is None); these entry points
 * serve this library's head-parallel layers (one process per GPU).  Every rank owns one region of device memory that its
 * peers map through a CUDA IPC handle.  A rank PUTS its pieces into its peers' regions with copy-engine transfers (no
 * multiprocessor is used, the transfers run beside the compute stream's kernels) and then raises one 32-bit flag per
 * peer; a consumer WAITS for its own flags with a one-warp kernel whose polling is bounded in time: when the limit
 * passes, the kernel records QB_ERR_TIMEOUT in the device status word (qb_read_device_status) and returns, so the
 * context stays usable.  Flags are counters that only grow: a waiter passes when `flag - value >= 0` (wrap-safe).
 *
 * qb_peer_alloc:  cudaMalloc + zero fill of `bytes`, and the 64-byte IPC handle other processes open.
 * qb_peer_open:   maps a peer's region into this process (peer access is enabled lazily by the driver).
 * qb_peer_close / qb_peer_free: the inverses.  Close every mapping before the owner frees its region.
 * qb_peer_put:    for every rank q < n with dst[q] != NULL: one cudaMemcpyAsync of `bytes` from
 *                 src + q * src_stride_bytes to dst[q] on `stream` (src_stride_bytes 0 sends the same piece to all),
 *                 issued in the order self+1, self+2, ... so that the ranks do not all start on the same peer; then one
 *                 kernel on `stream` that stores `value` to every flag[q] != NULL with system scope.  Stream order puts the
 *                 flag after the data.  With stream_of[q] != NULL the piece for rank q and its flag go on that stream
 *                 instead (one stream per destination lets several copy engines work at once); after_event != NULL
 *                 (a cudaEvent_t) makes every stream used wait for that event first: the producer of `src`.
 * qb_peer_wait:   one warp on `stream`; lane i < n polls flags[i] (this rank's own memory) until it reaches `value` or
 *                 `timeout_ms` passes.
 * qb_sum_partials: out[i] = fp16(sum over p < n_partials of partials[p * partial_stride + i]) for i < n, the sum taken
 *                 in fp32 in the order p = 0, 1, ...: the reduce half of the exchange on the receiving rank. */
#define QB_MAX_PEERS 16
typedef struct {
  const void* src;
  int64_t src_stride_bytes;
  int64_t bytes;
  void* dst[QB_MAX_PEERS];
  uint32_t* flag[QB_MAX_PEERS];
  void* stream_of[QB_MAX_PEERS];
  void* after_event;
  int32_t n;
  int32_t self;
  uint32_t value;
} qb_peer_put_args;
int qb_peer_alloc(int64_t bytes, void** ptr, unsigned char handle[64]);
int qb_peer_open(const unsigned char handle[64], void** ptr);
int qb_peer_close(void* ptr);
int qb_peer_free(void* ptr);
int qb_peer_put(const qb_peer_put_args* a, void* stream);
int qb_peer_wait(const uint32_t* flags, int32_t n, uint32_t value, int32_t timeout_ms, void* stream);
int qb_sum_partials(const void* partials, int32_t n_partials, int64_t partial_stride, void* out, int64_t n, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* QUAMBA_B200_H_ */
