/* C ABI of libembodiinfer_b200.so: the quantised-Linear hot path for NVIDIA B200 (sm_100a).
 *
 * Conventions (the same ones the reference's ctypes wrappers rely on,
 * embodiinfer/backend/cuda/quantization.py:33-66, embodiinfer/backend/cuda/native.py:119):
 *   - every pointer is a raw device pointer unless stated otherwise; `stream` is a cudaStream_t;
 *   - nothing is allocated, freed or synchronised: outputs and workspaces belong to the caller,
 *     so every entry point may be recorded into a CUDA graph after one warm-up call;
 *   - the return value is 0 on success, a negative B2_E_* code for a rejected argument, or a
 *     positive cudaError_t value reported by the launch;
 *   - scalars that must stay mutable under graph replay (scales) are read from device memory.
 *
 * Matrices are row-major.  bf16 is the 16-bit brain float, e4m3 the FP8 "fn" variant (max 448),
 * packed e2m1 holds two 4-bit codes per byte with the even column in the low nibble.
 */
#ifndef EMBODIINFER_B200_H
#define EMBODIINFER_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* 7: b2_attention_nvfp4.
 * 6: launches of at most 128 tokens may run on the cluster schedule (weights as the MMA's "A" operand, K split across a
 * thread-block cluster; B2_LINEAR_CLUSTER asks for it whenever it applies, B2_LINEAR_SINGLE_CTA opts out);
 * b2_gelu_table_range returns ranges on multiples of eight codes; FP8 launches accept 32 features per tile;
 * b2_attention_fp8; b2_linear_desc.rope (the attention preparation as the projection's epilogue).
 * 5: b2_attention.
 * 4: launches with more than 128 tokens run on pairs of SMs (B2_LINEAR_SINGLE_CTA opts out); unknown flag bits in
 * b2_linear_desc are rejected; the opt-in cluster split of K of version 3 (flag value 32) is gone.
 * 3: added the producers in front of the GEMMs (b2_norm_quant, b2_layer_norm_quant, b2_bhsd_quant, b2_normalize_frames,
 * b2_frames_to_patches, b2_resize_frames). */
#define B2_ABI_VERSION 7

/* ---- status codes ---------------------------------------------------------- */
#define B2_OK 0
#define B2_E_INVALID (-1)     /* null pointer, non-positive size, misaligned pointer */
#define B2_E_UNSUPPORTED (-2) /* shape outside what the kernel implements */
#define B2_E_DRIVER (-3)      /* tensor-map creation or driver entry point lookup failed */
#define B2_E_TOO_LARGE (-4)   /* size beyond a documented maximum */

/* ---- quantiser arithmetic flags ----------------------------------------------
 * The reference has two bit-exact quantiser arithmetics; both are implemented.
 *   spec T: the torch route   (backend/torch/fp8.py:66-73, backend/torch/nvfp4.py:28-46)
 *   spec C: the CUDA route    (backend/cuda/csrc/quantize.cu:38-104)
 */
#define B2_SPEC_T 0
#define B2_SPEC_C 1        /* fp32 quotient, hardware round-to-nearest-even e2m1, zero block -> code 0 */
#define B2_SCALAR_RCP 2    /* tensor / python-scalar evaluated as tensor * fp32(1/scalar), as ATen does on CUDA
                              and quantize.cu:54 does; without it a true division, as ATen does on CPU */
#define B2_DIVISOR_BF16 4  /* spec T FP8 only: round the scale to bf16 before dividing */
#define B2_CLAMP_TINY 8    /* scale = max(amax, FLT_MIN)/bound (nvfp4.py:38) instead of "1.0 when amax == 0" */
#define B2_GEGLU_TRUE_DIV 16 /* FP8 GELU*up epilogue divides by the scale (fusion.cu:21) instead of
                                multiplying by 1/scale (fusion.cu:87-92, the path every real shape takes) */

int b2_abi_version(void);

/* Number of bytes of zero-initialised device scratch b2_tensor_scale needs (it leaves them zero). */
#define B2_SCALE_SCRATCH_BYTES 8

/* Tensor amax -> scale = amax / bound, written to `scale` (device fp32).
 * Replaces cc_scale (backend/cuda/csrc/quantize.cu:116-125) and the amax lines of
 * fp8.py:70-71 / nvfp4.py:38.  `input` is bf16[count], 16-byte aligned.  `scratch` is
 * B2_SCALE_SCRATCH_BYTES of device memory that is zero before the first call; the kernel
 * restores it to zero, so calls on one stream may share it.  flags: B2_SCALAR_RCP, B2_CLAMP_TINY. */
int b2_tensor_scale(const void* input, int64_t count, float bound, int flags, void* scratch, void* scale,
                    void* stream);

/* Same result as b2_tensor_scale, for callers that cannot provide scratch memory and must not allocate:
 * a control loop working inside a fixed arena of device pointers owned by another runtime, or a server
 * that bans cudaMalloc once it is running because the call synchronises the device.  It has no
 * counterpart in the reference.  The scratch is a static device array of B2_STATIC_SCRATCH_BYTES inside
 * the library (held by every GPU that loads it, until the process exits).  Limits and rules:
 *   - count <= B2_STATIC_SCALE_MAX_COUNT elements, otherwise B2_E_TOO_LARGE;
 *   - the first call on each device looks up the array's device address (that device must be current);
 *     make that first call before starting any stream capture;
 *   - all calls on a GPU share the one array: calls that overlap on that GPU (two streams, two threads)
 *     race; calls ordered on one stream do not.  Nothing needs zeroing by the caller.
 * It allocates and frees nothing. */
#define B2_STATIC_SCRATCH_BYTES 16640
#define B2_STATIC_SCALE_MAX_COUNT 67108864
int b2_tensor_scale_static(const void* input, int64_t count, float bound, int flags, void* scale, void* stream);

/* bf16[count] -> e4m3[count] with the per-tensor scale read from device memory.
 * Replaces cc_fp8 (quantize.cu:127-133); spec T reproduces fp8.py:72.  flags: B2_SPEC_*, B2_DIVISOR_BF16. */
int b2_fp8_quantize(const void* input, void* output, const void* scale, int64_t count, int flags, void* stream);

/* bf16[rows, columns] -> packed e2m1 [rows, columns/2], e4m3 block scales in row-major order
 * (`scales`, [rows, columns/16], may be NULL) and in the 128x4-tile order the tensor core reads
 * (`blocked`, ceil(rows/128)*128 * ceil(columns/64)*4 bytes whose padding the caller zeroed once; may be
 * NULL).  `global` is the device fp32 global scale.  columns % 16 == 0.
 * Replaces cc_fp4 (quantize.cu:135-142) and nvfp4.quantize_weight + blocked_scales (nvfp4.py:14-46). */
int b2_nvfp4_quantize(const void* input, void* output, void* scales, void* blocked, const void* global, int rows,
                      int columns, int flags, void* stream);

/* h = bf16(bf16(gelu(gate)) * up) with GELU read from `table` (uint16[65536], indexed by the bf16 bit
 * pattern of gate), then stored as bf16 (bits 16), e4m3 (bits 8) or NVFP4 (bits 4).
 * gate/up are bf16 [rows, columns] with row stride `row_stride` elements (row_stride == columns for two
 * separate matrices; 2*columns with up == gate + columns for one packed [rows, 2*columns] matrix).
 * Replaces cc_geglu, cc_geglu_fp4, cc_geglu_packed and cc_geglu_bf16_strided
 * (backend/cuda/csrc/fusion.cu:109-200).  `scale` is the device fp32 calibrated scale (unused for 16 bits);
 * `scales`/`blocked` as in b2_nvfp4_quantize (4 bits only).  flags: B2_GEGLU_TRUE_DIV. */
int b2_geglu(const void* gate, const void* up, void* output, void* scales, void* blocked, const void* scale,
             int rows, int columns, int64_t row_stride, int bits, const void* table, int flags, void* stream);

/* ---- the tensor-core Linear ------------------------------------------------- */

#define B2_KIND_FP8 0   /* e4m3 x e4m3, per-tensor fp32 scales            (fp8.py:118-141, projection.py:155-163) */
#define B2_KIND_NVFP4 1 /* e2m1 x e2m1, ue4m3 scale per 16, fp32 globals  (nvfp4.py:96-123, projection.py:224-234) */

#define B2_EPI_LINEAR 0 /* out = act * weight^T (+bias)(+residual) */
#define B2_EPI_GEGLU 1  /* weight holds [gate; up] (2*features rows): out = GELU(act*gate^T) * (act*up^T) */
#define B2_EPI_GELU 2   /* out = GELU(act*weight^T + bias) through the table; bf16, or e4m3 at *out_scale (B2_OUT_FP8):
                           SigLIP fc1 + bias + tanh-GELU + the encoder of fc2's input (policies/pi05/inference/vision.py:441-576) */

#define B2_OUT_BF16 0
#define B2_OUT_FP8 1    /* GEGLU, GELU: e4m3 at *out_scale                   (fusion.cu:64-107) */
#define B2_OUT_NVFP4 2  /* GEGLU only: packed e2m1 + block scales at *out_scale (fusion.cu:31-62) */

#define B2_LINEAR_ROUND_SCALE_BF16 1 /* NVFP4 registry route: y = bf16(bf16(acc) * bf16(g_a*g_w))
                                        (nvfp4.py:120, quantize.cu:106-114) instead of bf16(acc*g_a*g_w) */

#define B2_LINEAR_PAIRED_GATE_UP_SCALES 4 /* GEGLU with NVFP4 operands: `weight_scales` is the 128x4-tile layout of the
                                            block scales with their ROWS reordered so that rows [128t, 128t+64) are gate
                                            features [64t, 64t+64) and rows [128t+64, 128t+128) the up features of the same
                                            range.  Each 64-feature tile then needs one scale block and one MMA per K step
                                            instead of two of each.  The weight codes keep the bundle order (gate, then up). */

#define B2_LINEAR_STREAM_TOKENS 8 /* tuning aid: always load the token tile with every K stage.  By default a CTA keeps its
                                     128-token tile (all of K) and the token scales on chip whenever they fit and it computes
                                     several feature tiles of that token tile; results are identical either way. */
#define B2_LINEAR_SINGLE_CTA 64 /* tuning / test aid: never use the paired schedule.  In the paired schedule 256-token tiles run on
                                  pairs of SMs (two CTAs of a thread-block cluster, `tcgen05.mma.cta_group::2`): each CTA loads its
                                  128 token rows and half of the weight tile.  The library picks it when there are more than 128
                                  tokens and the 256-row tiles add no padding over 128-row tiles (or there are at least 2048 tokens).
                                  The accumulation order along K is the same in both schedules: results are identical either way. */
#define B2_LINEAR_PAIRS 128 /* tuning / test aid: use the paired schedule whenever it applies (more than 128 tokens, no split K,
                               bundle-order scale layout), whatever the padding */
#define B2_LINEAR_CLUSTER 256 /* tuning / test aid: use the cluster schedule whenever it applies (at most 128 tokens, no feature
                                 tile asked for; gated NVFP4 only with B2_LINEAR_PAIRED_GATE_UP_SCALES).  There the 128 rows of the
                                 MMA's "A" operand are 128 features (64 gate + 64 up), the tokens are its columns, and the K of a
                                 feature tile is cut across the 1, 2, 4 or 8 CTAs of a thread-block cluster, which exchange fp32
                                 partial sums through distributed shared memory and add them in a fixed order.  The library picks
                                 it by an estimate of both schedules' times (few tokens, long K); B2_LINEAR_SINGLE_CTA opts out.
                                 K is summed in a different order than in the tile schedules: results agree to fp32 rounding. */

/* The attention preparation of b2_rope_split as the epilogue of the packed QKV projection (b2_linear_desc.rope); fields as
 * in b2_rope_split. */
typedef struct b2_rope_desc {
    const void* sine;
    const void* cosine;
    void* q_out;
    void* k_out;
    void* v_out;
    int64_t factor_batch_stride;
    int32_t batch, tokens, heads, kv_heads, head_dim, kv_capacity, kv_offset;
} b2_rope_desc;

typedef struct b2_linear_desc {
    int32_t kind;        /* B2_KIND_* */
    int32_t epilogue;    /* B2_EPI_* */
    int32_t out_format;  /* B2_OUT_* */
    int32_t flags;       /* B2_LINEAR_ROUND_SCALE_BF16 | B2_LINEAR_PAIRED_GATE_UP_SCALES | B2_LINEAR_STREAM_TOKENS | B2_LINEAR_SINGLE_CTA | B2_LINEAR_PAIRS | B2_LINEAR_CLUSTER | B2_GEGLU_TRUE_DIV; any other bit: B2_E_INVALID */
    int32_t tokens;      /* M: rows of the activation matrix */
    int32_t features;    /* N: output width (GEGLU: the weight has 2*features rows, gate first) */
    int32_t width;       /* K: inner dimension; K % 16 == 0 (FP8), K % 64 == 0 (NVFP4) */
    int32_t feature_tile; /* output features per tile: 0 = choose; LINEAR 64/128/192/256 (FP8 also 32), GEGLU 64/128 */
    int32_t gelu_lo;      /* GEGLU: range of bf16 magnitude codes from b2_gelu_table_range, or 0, 0 */
    int32_t gelu_hi;
    const void* act;           /* e4m3 [M, K] or packed e2m1 [M, K/2] */
    const void* act_scales;    /* NVFP4: block scales of act in 128x4-tile order */
    const void* act_scale;     /* device fp32: per-tensor scale (FP8) or global scale (NVFP4) */
    const void* weight;        /* e4m3 [rows, K] or packed e2m1 [rows, K/2] */
    const void* weight_scales; /* NVFP4: block scales of weight in 128x4-tile order */
    const void* weight_scale;  /* device fp32 */
    const void* weight_scale_up; /* GEGLU: device fp32 scale of the up rows when gate and up were quantised
                                    separately; NULL = weight_scale covers both */
    const void* bias;          /* bf16 [N] or NULL (LINEAR only) */
    const void* residual;      /* bf16 [M, N] or NULL (LINEAR only): out = bf16(y + residual) */
    const void* gelu_table;    /* uint16[65536] (GEGLU only) */
    const void* out_scale;     /* device fp32 the epilogue quantises at (B2_OUT_FP8 / B2_OUT_NVFP4) */
    void* out;                 /* bf16 [M, N] | e4m3 [M, N] | packed e2m1 [M, N/2] */
    void* out_scales;          /* B2_OUT_NVFP4: row-major block scales [M, N/16] or NULL */
    void* out_blocked;         /* B2_OUT_NVFP4: block scales in 128x4-tile order (padding zeroed by caller) */
    void* status;              /* device uint32 or NULL: set nonzero if a bounded device-side wait expired */
    void* workspace;           /* NULL, or device scratch for split K (16-byte aligned, ZERO before its first use; every
                                  launch leaves its first 1024 bytes (the ticket words) zero again, so
                                  launches that follow one another on a stream may share it) */
    int64_t workspace_bytes;   /* size of `workspace`; split K is used only when b2_linear_workspace_bytes(desc) fits */
    const b2_rope_desc* rope;  /* NULL, or: this launch is a packed QKV projection whose result goes through b2_rope_split's
                                  arithmetic in the epilogue -- rotated queries to q_out, rotated keys and plain values into the
                                  key/value buffers -- instead of being stored to `out` (ignored, may be NULL).  Same bits as
                                  b2_linear followed by b2_rope_split, one launch less.  Cluster schedule only: B2_KIND_FP8,
                                  B2_EPI_LINEAR, no bias, no residual, tokens == batch * rope->tokens <= 128, head_dim 256,
                                  features == (heads + 2 kv_heads) * 256; anything else: B2_E_UNSUPPORTED. */
} b2_linear_desc;

/* Attention preparation after a packed QKV projection (the steps between the projection and the attention in
 * embodiinfer/policies/pi05/modeling_pi05.py:924-1010: split, rotary embedding, layout change, key/value cache
 * write; rotation arithmetic of embodiinfer/backend/torch/rotary.py:24-27, contract "fp32_rope_bf16_output").
 *   qkv     bf16 [batch*tokens, (heads + 2*kv_heads) * head_dim]: per token q heads, then k heads, then v heads
 *   sine, cosine  fp32 [tokens, head_dim/2] (factor_batch_stride = 0) or [batch, tokens, head_dim/2]
 *                 (factor_batch_stride = tokens*head_dim/2)
 *   q_out   bf16 [batch, heads, tokens, head_dim]              rotated queries
 *   k_out, v_out  bf16 [batch, kv_heads, kv_capacity, head_dim]: rotated keys and plain values are written at
 *                 token positions [kv_offset, kv_offset + tokens); other positions are left untouched
 * head_dim must be a multiple of 16; all pointers 16-byte aligned. */
int b2_rope_split(const void* qkv, const void* sine, const void* cosine, void* q_out, void* k_out, void* v_out,
                  int32_t batch, int32_t tokens, int32_t heads, int32_t kv_heads, int32_t head_dim,
                  int64_t factor_batch_stride, int32_t kv_capacity, int32_t kv_offset, void* stream);

/* Multi-query attention of the Gemma-shaped towers, unmasked:
 *   out[b, h, t, :] = softmax(q[b, h, t, :] . k[b, :, :]^T / sqrt(head_dim)) v[b, :, :]
 * It is the attention between the QKV projection and the output projection
 * (embodiinfer/backend/torch/attention.py:97-106, SDPAAttention: scaled_dot_product_attention with one key/value head
 * shared by all query heads), and for a ten-query chunk over prefix + chunk keys the job of
 * embodiinfer/backend/cuda/csrc/mqa_decode_attention.cu:170-393.
 *   q    bf16 [batch, heads, queries, head_dim]   (b2_rope_split's q_out)
 *   k, v bf16 [batch, 1, keys, head_dim]           (b2_rope_split's k_out / v_out with kv_capacity == keys)
 *   out  bf16 [batch, heads, queries, head_dim]   (what b2_bhsd_quant reads)
 * head_dim must be 256 (B2_E_UNSUPPORTED otherwise); all pointers 16-byte aligned.  Scores and the output accumulate in
 * fp32; probabilities enter the second product as bf16, as in torch's flash kernels.  A launch of few 128-row tiles (a handful
 * of ten-query chunks) cuts the keys of a tile across a thread-block cluster of up to 16 CTAs and merges the partial rows
 * (fp16 scaled per row by a power of two, with fp32 maxima and sums) in a fixed order.  `status` as in b2_linear_desc
 * (NULL allowed). */
int b2_attention(const void* q, const void* k, const void* v, void* out, int32_t batch, int32_t heads, int32_t queries,
                 int32_t keys, int32_t head_dim, void* status, void* stream);

/* The same attention with the output written straight as the e4m3 rows of the output projection: `codes`
 * [batch * queries, heads * head_dim] = e4m3(bf16(out[b, h, t, :]) * multiplier) at row b * queries + t, columns of head h --
 * bit-identical to b2_attention followed by b2_bhsd_quant (bits 8, scale_value = multiplier), one launch less on the
 * expert's chain of short kernels.  multiplier: 448 / calibrated maximum, finite and positive. */
int b2_attention_fp8(const void* q, const void* k, const void* v, void* codes, float multiplier, int32_t batch, int32_t heads,
                     int32_t queries, int32_t keys, int32_t head_dim, void* status, void* stream);

/* The same attention with the output written as the NVFP4 rows of the output projection: `codes` packed e2m1
 * [batch * queries, heads * head_dim / 2], `blocked` their e4m3 block scales in 128 x 4 tile order (padding zeroed by the
 * caller), `scales` the same block scales row-major [batch * queries, heads * head_dim / 16] or NULL -- bit-identical to
 * b2_attention followed by b2_bhsd_quant (bits 4, scale_value = global_scale).  global_scale: the projection's static
 * global scale (calibrated maximum / (448 * 6)), finite and positive. */
int b2_attention_nvfp4(const void* q, const void* k, const void* v, void* codes, void* scales, void* blocked, float global_scale,
                       int32_t batch, int32_t heads, int32_t queries, int32_t keys, int32_t head_dim, void* status, void* stream);

/* RMSNorm (+ residual update, + adaptive modulation) fused with the activation encoder: the step in front of
 * every quantised projection.  Replaces cc_norm_quant and cc_norm_quant_reduce
 * (embodiinfer/backend/cuda/csrc/norm_quant.cu:91-112, 517-562; bound by NormQuantPlan.normalize /
 * residual_normalize, embodiinfer/backend/cuda/norm_quant.py:139-303) and the bf16 result of the strict
 * normalisation (contract "torch_rmsnorm_bf16_rounding", embodiinfer/backend/torch/normalization.py:49-103).
 *
 * Per row (token), in the reference's fp32 arithmetic and rounding points:
 *   r   = update == NULL ? input : bf16(input + (update_gate ? bf16(update * update_gate[batch]) : update))
 *   inv = rsqrtf(mean + 1e-6), mean = mean[row] when given, else sum(r*r) * fp32(1/columns), the sum taken
 *         in the reference kernels' order (columns 1024 and 2048: 8 consecutive columns per lane, then a
 *         butterfly over 32 lanes and over the warps; other widths: 256 strided lanes, then a halving tree)
 *   y   = bf16(modulation ? (r*inv) * (1 + m_scale) + m_shift : (r*inv) * (1 + scale))
 *   bits 16: output = y (bf16)
 *   bits 8 : output = e4m3(y * fp32(1 / *global))  (mean == NULL)  or  e4m3(y / *global)  (mean given)
 *   bits 4 : NVFP4 spec C of y at *global: packed e2m1, row-major block scales (`scales`, may be NULL) and
 *            the 128x4-tile layout (`blocked`; padding bytes are the caller's to zero)
 * `residual` (may be NULL) receives r; `gate` (may be NULL) receives bf16(modulation[:, 2*columns:]) per batch
 * entry; `inverse` (may be NULL) receives inv per row (test hook: rsqrtf is the one step a CPU cannot
 * restate bit-exactly).  `modulation` is fp32 [rows/tokens, 3*columns] = scale | shift | gate.
 * columns % 64 == 0, columns <= 8192, rows % tokens == 0; bf16 pointers 16-byte aligned.
 * flags: B2_NORM_RESIDUAL_EVICT_LAST stores `residual` with an L2 evict-last policy (norm_quant.cu:370-379). */
#define B2_NORM_RESIDUAL_EVICT_LAST 1
typedef struct b2_norm_desc {
    const void* input;       /* bf16 [rows, columns] */
    const void* update;      /* bf16 [rows, columns] or NULL */
    const void* update_gate; /* bf16 [rows/tokens, columns] or NULL */
    const void* scale;       /* fp32 [columns], RMSNorm weight without the +1; ignored when modulation != NULL */
    const void* modulation;  /* fp32 [rows/tokens, 3*columns] or NULL */
    const void* mean;        /* fp32 [rows] mean of squares, or NULL: reduce in the kernel */
    const void* global;      /* device fp32: per-tensor scale (bits 8) or NVFP4 global scale (bits 4); NULL for bits 16 */
    void* residual;          /* bf16 [rows, columns] or NULL */
    void* output;            /* bf16 [rows, columns] | e4m3 [rows, columns] | packed e2m1 [rows, columns/2] */
    void* scales;            /* bits 4: e4m3 [rows, columns/16] or NULL */
    void* blocked;           /* bits 4: block scales in 128x4-tile order */
    void* gate;              /* bf16 [rows/tokens, columns] or NULL (modulation only) */
    void* inverse;           /* fp32 [rows] or NULL */
    int32_t rows, columns, tokens, bits, flags;
} b2_norm_desc;
int b2_norm_quant(const b2_norm_desc* desc, void* stream);

/* LayerNorm (+ residual update) fused with the activation encoder, for the SigLIP tower.  Replaces
 * cc_layer_norm_fp8 and cc_layer_norm_fp4 (embodiinfer/backend/cuda/csrc/norm_quant.cu:678-687, 922-931; called
 * from embodiinfer/policies/pi05/inference/vision.py:303-546).  Per row, every step a separate fp32 rounding
 * (the reference compiles these kernels without fused multiply-add):
 *   r    = update == NULL ? input : bf16(input + update)                     (`residual`, may be NULL, receives r)
 *   mean = sum(r) / columns, var = max(0, sum(r*r) / columns - mean*mean), inv = rsqrtf(var + 1e-6), sums in the
 *          reference kernels' order (8 columns per lane in pairs, 32-lane butterfly, butterfly over the warps
 *          of a 160-thread block when columns <= 1152, else of a 256-thread block)
 *   y    = bf16((((r - mean) * inv) * weight) + bias)                        weight, bias: bf16 [columns]
 *   bits 16: output = y;  bits 8: output = e4m3(y * scale_value) (scale_value = 448 / calibrated maximum, the
 *   reciprocal of the activation scale, as the reference passes it);  bits 4: NVFP4 spec C of y at the global
 *   scale `scale_value`: packed e2m1, `blocked` scales in 128x4-tile order, `scales` (may be NULL) row-major.
 * `statistics` (may be NULL) receives fp32 [rows, 2] = mean, inv (test hook, see b2_norm_quant).
 * columns % 16 == 0, columns <= 2048; bf16 pointers 16-byte aligned. */
int b2_layer_norm_quant(const void* input, const void* update, const void* weight, const void* bias, void* residual,
                        void* output, void* scales, void* blocked, void* statistics, float scale_value, int32_t rows,
                        int32_t columns, int32_t bits, void* stream);

/* Attention output [batch, heads, tokens, head_dim] (any batch / head / token strides, head_dim contiguous) ->
 * encoded rows [batch*tokens, heads*head_dim] for the output projection: the transpose fused with the activation
 * encoder.  Replaces cc_bhsd_fp8 and cc_bhsd_fp4 (embodiinfer/backend/cuda/csrc/norm_quant.cu:720-731, 785-795;
 * bound in embodiinfer/backend/cuda/norm_quant.py:49-78).
 *   bits 8 : e4m3(x * scale_value), scale_value = the reciprocal of the activation scale (by value, as the
 *            reference passes it)
 *   bits 4 : NVFP4 spec C at the global scale `scale_value`: packed e2m1, `blocked` scales in 128x4-tile order
 *            (padding is the caller's to zero), `scales` (may be NULL) row-major
 *   bits 16: bf16 copy in the new layout
 * Strides are in elements.  head_dim % 8 == 0 (16 for bits 4); input and output 16-byte aligned, strides
 * multiples of 8 elements. */
int b2_bhsd_quant(const void* input, void* output, void* scales, void* blocked, float scale_value, int64_t stride_b,
                  int64_t stride_h, int64_t stride_s, int32_t batch, int32_t heads, int32_t tokens, int32_t head_dim,
                  int32_t bits, void* stream);

/* Camera frames uint8 [cameras, height*width, 3] -> fp32 planes [cameras, 3, height*width] holding
 * (x / 255) * 2 - 1, each step rounded separately in fp32.  Replaces cc_normalize_frames
 * (embodiinfer/backend/cuda/csrc/camera_frames.cu:107-115; bound in embodiinfer/backend/cuda/camera_frames.py:45-61). */
int b2_normalize_frames(const void* frames, void* images, int32_t cameras, int32_t pixels, void* stream);

/* OpenPI's resize_with_pad on the device: uint8 frames [cameras, height, width, 3] are resampled to
 * [out_height, out_width] with Pillow's two-pass 8-bit bilinear filter (22-bit fixed-point taps, a byte clamp after
 * each pass), placed at (top, left) on a black [canvas_height, canvas_width] canvas and written as fp32 planes
 * [cameras, 3, canvas_height, canvas_width] of (x / 255) * 2 - 1.  Replaces cc_resize_frames
 * (embodiinfer/backend/cuda/csrc/camera_frames.cu:90-105; bound by FrameResize,
 * embodiinfer/backend/cuda/camera_frames.py:93-160) in one launch and without its `rows` scratch.
 * Device int32 tables, as the reference's host code builds them: `*_bounds` [out, 2] = first source index and tap
 * count per output index, `*_weights` [out, *_taps] fixed-point taps (row_* for the horizontal axis, column_* for
 * the vertical one). */
int b2_resize_frames(const void* frames, void* images, const void* row_bounds, const void* row_weights, int32_t row_taps,
                     const void* column_bounds, const void* column_weights, int32_t column_taps, int32_t cameras,
                     int32_t height, int32_t width, int32_t out_height, int32_t out_width, int32_t canvas_height,
                     int32_t canvas_width, int32_t top, int32_t left, void* stream);

/* Camera frames uint8 [cameras, height, width, 3] -> bf16 patch rows [cameras * (height/patch) * (width/patch),
 * 3*patch*patch], row = (camera, patch row, patch column), column = (channel, y in patch, x in patch), value =
 * bf16((x / 255) * 2 - 1): the normalisation above followed by the cast and the patch gather of the SigLIP patch
 * embedding (embodiinfer/policies/pi05/inference/vision.py:593-602) in one launch, bit-identical to those steps.
 * height % patch == 0, width % patch == 0, (3*patch*patch) % 4 == 0; `patches` 8-byte aligned. */
int b2_frames_to_patches(const void* frames, void* patches, int32_t cameras, int32_t height, int32_t width, int32_t patch,
                         void* stream);

/* Device scratch a launch described by `desc` could use, in bytes (0: it would not split K; only B2_EPI_LINEAR
 * launches split).  With few
 * tiles (M = 10*B tokens against 148 SMs) the library cuts K into up to 16 ranges computed by different CTAs;
 * the CTA that finishes a tile last adds the fp32 partial sums in a fixed order (results do not depend on
 * timing) and runs the epilogue.  Without a workspace the same launch runs unsplit.  Pointer fields of
 * `desc` are not dereferenced.  No reference counterpart (cuBLASLt manages its own workspace behind
 * F.scaled_mm). */
int64_t b2_linear_workspace_bytes(const b2_linear_desc* desc);

/* Which part of a GELU table needs to be looked up.  `host_table` is a HOST copy of the uint16[65536]
 * table.  On success *lo and *hi bound the bf16 magnitude codes [lo, hi) outside which the table
 * provably equals a closed form for every finite normal input: bf16(x/2) below lo; x (positive) or -0
 * (negative) from hi upward.  b2_linear then keeps only [lo, hi) of the table, for both signs, in shared
 * memory and evaluates the closed forms elsewhere, which is bit-identical to indexing the full table.
 * Returns B2_E_UNSUPPORTED (and 0, 0) when the table has no such structure or the range is wider than
 * 4096 codes; b2_linear then reads the full table from global memory.  The tanh-approximated GELU's closed forms
 * hold outside [0x3b4b, 0x40a2) (|x| in [3.1e-3, 5.06)); the function returns lo lowered by ten binades (0x364b)
 * and hi raised by four (0x42a2, |x| = 81), which is as valid and keeps nearly every gate value inside the range (one
 * straight-line path per warp, also for heavy-tailed activations).  Host-only; no reference counterpart (the reference
 * always gathers from the 128 KiB table, fusion.cu:5-10). */
int b2_gelu_table_range(const void* host_table, int32_t* lo, int32_t* hi);

/* One launch: TMA-staged operands, tcgen05 MMA into TMEM, fused epilogue.
 * LINEAR needs N % 8 == 0; GEGLU needs N % 16 == 0 (N % 128 == 0 for NVFP4 operands).
 * bias, residual and out must be 16-byte aligned.
 * Replaces the library GEMM + separate elementwise launches behind fp8.native_linear (fp8.py:118-141),
 * nvfp4._native_linear (nvfp4.py:96-123), Projection.apply (projection.py:108-235) and, for GEGLU,
 * the two GEMMs + cc_geglu/cc_geglu_fp4 of MlpPlan (policies/pi05/inference/mlp.py:481-501).
 * `desc` is host memory and is read before the call returns. */
int b2_linear(const b2_linear_desc* desc, void* stream);

#ifdef __cplusplus
}
#endif

#endif /* EMBODIINFER_B200_H */
