// extern "C" surface of libembodiinfer_b200.so: argument checks, then the launchers.
// Declarations and per-entry documentation live in include/embodiinfer_b200.h.
#include "common.cuh"

#include <cstring>

namespace b2 {
int run_linear(const b2_linear_desc* desc, cudaStream_t stream, int64_t* workspace_need = nullptr);
int launch_attention(const void* q, const void* k, const void* v, void* out, void* codes, float multiplier, void* block_scales,
                     void* blocked, float global_scale, int batch, int heads, int queries, int keys, int head_dim, void* status,
                     cudaStream_t stream);
int launch_rope_split(const void* qkv, const void* sine, const void* cosine, void* q_out, void* k_out, void* v_out, int batch,
                      int tokens, int heads, int kv_heads, int head_dim, int64_t factor_batch_stride, int kv_capacity,
                      int kv_offset, cudaStream_t stream);
int launch_geglu(const void* gate, const void* up, void* output, void* scales, void* blocked, const void* scale,
                 int rows, int columns, int64_t row_stride, int bits, const void* table, int flags,
                 cudaStream_t stream);
int launch_norm_quant(const b2_norm_desc* desc, cudaStream_t stream);
int launch_resize_frames(const void* frames, void* images, const void* row_bounds, const void* row_weights, int row_taps,
                         const void* column_bounds, const void* column_weights, int column_taps, int cameras, int height,
                         int width, int out_height, int out_width, int canvas_height, int canvas_width, int top, int left,
                         cudaStream_t stream);
int launch_normalize_frames(const void* frames, void* images, int cameras, int pixels, cudaStream_t stream);
int launch_frames_to_patches(const void* frames, void* patches, int cameras, int height, int width, int patch,
                             cudaStream_t stream);
int launch_bhsd_quant(const void* input, void* output, void* scales, void* blocked, float scale_value, int64_t stride_b,
                      int64_t stride_h, int64_t stride_s, int batch, int heads, int tokens, int head_dim, int bits,
                      cudaStream_t stream);
int launch_layer_norm_quant(const void* input, const void* update, const void* weight, const void* bias, void* residual,
                            void* output, void* scales, void* blocked, void* statistics, float scale_value, int rows,
                            int columns, int bits, cudaStream_t stream);
int launch_tensor_scale_static(const void* input, int64_t count, float bound, int flags, void* scale,
                               cudaStream_t stream);
}  // namespace b2

static bool is_aligned(const void* pointer, uintptr_t bytes) {
    return (reinterpret_cast<uintptr_t>(pointer) & (bytes - 1)) == 0;
}

extern "C" {

int b2_abi_version(void) { return B2_ABI_VERSION; }

int b2_tensor_scale(const void* input, int64_t count, float bound, int flags, void* scratch, void* scale,
                    void* stream) {
    if (input == nullptr || scratch == nullptr || scale == nullptr || count <= 0 || !(bound > 0.0f)) return B2_E_INVALID;
    if (!is_aligned(input, 16) || !is_aligned(scratch, 4) || !is_aligned(scale, 4)) return B2_E_INVALID;
    return b2::launch_tensor_scale(input, count, bound, flags, scratch, scale, static_cast<cudaStream_t>(stream));
}

int b2_tensor_scale_static(const void* input, int64_t count, float bound, int flags, void* scale, void* stream) {
    if (input == nullptr || scale == nullptr || count <= 0 || !(bound > 0.0f)) return B2_E_INVALID;
    if (!is_aligned(input, 16) || !is_aligned(scale, 4)) return B2_E_INVALID;
    return b2::launch_tensor_scale_static(input, count, bound, flags, scale, static_cast<cudaStream_t>(stream));
}

int b2_fp8_quantize(const void* input, void* output, const void* scale, int64_t count, int flags, void* stream) {
    if (input == nullptr || output == nullptr || scale == nullptr || count <= 0) return B2_E_INVALID;
    if (!is_aligned(input, 16) || !is_aligned(output, 8)) return B2_E_INVALID;
    return b2::launch_fp8_encode(input, output, scale, count, flags, static_cast<cudaStream_t>(stream));
}

int b2_nvfp4_quantize(const void* input, void* output, void* scales, void* blocked, const void* global, int rows,
                      int columns, int flags, void* stream) {
    if (input == nullptr || output == nullptr || global == nullptr || rows <= 0 || columns <= 0) return B2_E_INVALID;
    if (columns % 16 != 0) return B2_E_UNSUPPORTED;
    if (!is_aligned(input, 16) || !is_aligned(output, 4)) return B2_E_INVALID;
    if ((scales != nullptr && !is_aligned(scales, 4)) || (blocked != nullptr && !is_aligned(blocked, 4)))
        return B2_E_INVALID;
    return b2::launch_nvfp4_encode(input, output, scales, blocked, global, rows, columns, flags,
                                   static_cast<cudaStream_t>(stream));
}

int b2_geglu(const void* gate, const void* up, void* output, void* scales, void* blocked, const void* scale,
             int rows, int columns, int64_t row_stride, int bits, const void* table, int flags, void* stream) {
    if (gate == nullptr || output == nullptr || table == nullptr || rows <= 0 || columns <= 0) return B2_E_INVALID;
    if (row_stride < columns) return B2_E_INVALID;
    if (bits != 4 && bits != 8 && bits != 16) return B2_E_UNSUPPORTED;
    if (bits != 16 && scale == nullptr) return B2_E_INVALID;
    return b2::launch_geglu(gate, up, output, scales, blocked, scale, rows, columns, row_stride, bits, table, flags,
                            static_cast<cudaStream_t>(stream));
}

static uint16_t host_bf16(float value) {
    uint32_t bits;
    memcpy(&bits, &value, 4);
    if ((bits & 0x7fffffffu) > 0x7f800000u) return 0x7fc0;
    return uint16_t((bits + 0x7fffu + ((bits >> 16) & 1u)) >> 16);
}

int b2_gelu_table_range(const void* host_table, int32_t* lo, int32_t* hi) {
    if (host_table == nullptr || lo == nullptr || hi == nullptr) return B2_E_INVALID;
    const uint16_t* table = static_cast<const uint16_t*>(host_table);
    *lo = *hi = 0;
    const int first = 0x80, last = 0x7f80;        // normal finite magnitudes
    int low = first;
    for (; low < last; ++low) {
        const uint32_t word = uint32_t(low) << 16;
        float x;
        memcpy(&x, &word, 4);
        if (table[low] != host_bf16(0.5f * x) || table[0x8000 + low] != host_bf16(-0.5f * x)) break;
    }
    int high = last;
    for (; high > low; --high)
        if (table[high - 1] != high - 1 || table[0x8000 + high - 1] != 0x8000) break;
    if (high - low > 4096) return B2_E_UNSUPPORTED;
    if (high == low) high = low + 1 <= last ? low + 1 : low;   // keep a non-empty range so the closed forms stay enabled
    // Any wider range is as valid (inside it the table itself is read).  Ten more binades below `low` cost 5 KB of
    // shared memory and make a gate outside the range a one-in-a-million event, so that a warp's look-ups stay on the
    // straight-line path: with the tight range a quarter of a percent of Gaussian gates fall below it, which sent
    // three warps in four through the slow general path as well.
    constexpr int MARGIN = 1280;
    const int widened = low - MARGIN > first ? low - MARGIN : first;
    if (high - widened <= 4096) low = widened;
    // And four binades above `high` (1 KB more): one gate in a hundred of a heavy-tailed activation lies beyond
    // the point where GELU(x) = x in bf16 (about 5), and a single such value among the 512 of a warp's unit is enough
    // to send the whole warp through the general path.
    constexpr int MARGIN_ABOVE = 512;
    const int raised = high + MARGIN_ABOVE < last ? high + MARGIN_ABOVE : last;
    if (raised - low <= 4096) high = raised;
    // Both ends on a multiple of eight codes (16 bytes) when that still fits: a kernel can then bring each half of the
    // range into shared memory with one bulk copy instead of a load per entry.
    const int low8 = low & ~7, high8 = (high + 7) & ~7;
    if (low8 >= first && high8 <= last && high8 - low8 <= 4096) {
        low = low8;
        high = high8;
    }
    *lo = low;
    *hi = high;
    return B2_OK;
}

int b2_linear(const b2_linear_desc* desc, void* stream) {
    return b2::run_linear(desc, static_cast<cudaStream_t>(stream));
}

int b2_attention(const void* q, const void* k, const void* v, void* out, int32_t batch, int32_t heads, int32_t queries,
                 int32_t keys, int32_t head_dim, void* status, void* stream) {
    if (q == nullptr || k == nullptr || v == nullptr || out == nullptr) return B2_E_INVALID;
    if (batch <= 0 || heads <= 0 || queries <= 0 || keys <= 0 || head_dim <= 0) return B2_E_INVALID;
    const uintptr_t alignment = reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v) |
                                reinterpret_cast<uintptr_t>(out);
    if (alignment & 15u) return B2_E_INVALID;
    return b2::launch_attention(q, k, v, out, nullptr, 1.0f, nullptr, nullptr, 1.0f, batch, heads, queries, keys, head_dim, status, static_cast<cudaStream_t>(stream));
}

int b2_attention_fp8(const void* q, const void* k, const void* v, void* codes, float multiplier, int32_t batch, int32_t heads,
                     int32_t queries, int32_t keys, int32_t head_dim, void* status, void* stream) {
    if (q == nullptr || k == nullptr || v == nullptr || codes == nullptr) return B2_E_INVALID;
    if (batch <= 0 || heads <= 0 || queries <= 0 || keys <= 0 || head_dim <= 0) return B2_E_INVALID;
    if (!(multiplier > 0.0f) || multiplier > 3.0e38f) return B2_E_INVALID;
    const uintptr_t alignment = reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v) |
                                reinterpret_cast<uintptr_t>(codes);
    if (alignment & 15u) return B2_E_INVALID;
    return b2::launch_attention(q, k, v, nullptr, codes, multiplier, nullptr, nullptr, 1.0f, batch, heads, queries, keys, head_dim, status, static_cast<cudaStream_t>(stream));
}

int b2_attention_nvfp4(const void* q, const void* k, const void* v, void* codes, void* scales, void* blocked, float global_scale,
                       int32_t batch, int32_t heads, int32_t queries, int32_t keys, int32_t head_dim, void* status, void* stream) {
    if (q == nullptr || k == nullptr || v == nullptr || codes == nullptr || blocked == nullptr) return B2_E_INVALID;
    if (batch <= 0 || heads <= 0 || queries <= 0 || keys <= 0 || head_dim <= 0) return B2_E_INVALID;
    if (!(global_scale > 0.0f) || global_scale > 3.0e38f) return B2_E_INVALID;
    const uintptr_t alignment = reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v) |
                                reinterpret_cast<uintptr_t>(codes);
    if (alignment & 15u) return B2_E_INVALID;
    return b2::launch_attention(q, k, v, nullptr, codes, 1.0f, scales, blocked, global_scale, batch, heads, queries, keys, head_dim, status,
                                static_cast<cudaStream_t>(stream));
}

int b2_rope_split(const void* qkv, const void* sine, const void* cosine, void* q_out, void* k_out, void* v_out,
                  int32_t batch, int32_t tokens, int32_t heads, int32_t kv_heads, int32_t head_dim,
                  int64_t factor_batch_stride, int32_t kv_capacity, int32_t kv_offset, void* stream) {
    if (qkv == nullptr || sine == nullptr || cosine == nullptr || q_out == nullptr || k_out == nullptr || v_out == nullptr)
        return B2_E_INVALID;
    if (batch <= 0 || tokens <= 0 || heads <= 0 || kv_heads <= 0 || head_dim <= 0 || kv_offset < 0 ||
        kv_offset + tokens > kv_capacity || factor_batch_stride < 0)
        return B2_E_INVALID;
    if (head_dim % 16 != 0) return B2_E_UNSUPPORTED;
    const uintptr_t alignment = reinterpret_cast<uintptr_t>(qkv) | reinterpret_cast<uintptr_t>(q_out) |
                                reinterpret_cast<uintptr_t>(k_out) | reinterpret_cast<uintptr_t>(v_out);
    if (alignment & 15u) return B2_E_INVALID;
    return b2::launch_rope_split(qkv, sine, cosine, q_out, k_out, v_out, batch, tokens, heads, kv_heads, head_dim,
                                 factor_batch_stride, kv_capacity, kv_offset, static_cast<cudaStream_t>(stream));
}

int b2_norm_quant(const b2_norm_desc* desc, void* stream) {
    if (desc == nullptr || desc->input == nullptr || desc->output == nullptr) return B2_E_INVALID;
    if (desc->rows <= 0 || desc->columns <= 0 || desc->tokens <= 0 || desc->rows % desc->tokens != 0) return B2_E_INVALID;
    if (desc->bits != 4 && desc->bits != 8 && desc->bits != 16) return B2_E_UNSUPPORTED;
    if (desc->columns % 64 != 0) return B2_E_UNSUPPORTED;
    if (desc->columns > 8192) return B2_E_TOO_LARGE;
    if (desc->flags & ~B2_NORM_RESIDUAL_EVICT_LAST) return B2_E_INVALID;
    if (desc->modulation == nullptr && desc->scale == nullptr) return B2_E_INVALID;
    if (desc->modulation == nullptr && desc->gate != nullptr) return B2_E_INVALID;
    if (desc->update == nullptr && desc->update_gate != nullptr) return B2_E_INVALID;
    if (desc->mean != nullptr && desc->update != nullptr) return B2_E_INVALID;
    if (desc->bits != 16 && desc->global == nullptr) return B2_E_INVALID;
    if (desc->bits == 4 && desc->blocked == nullptr) return B2_E_INVALID;
    const void* vectors[] = {desc->input, desc->update, desc->update_gate, desc->scale, desc->modulation,
                             desc->residual, desc->output, desc->gate};
    for (const void* pointer : vectors)
        if (!is_aligned(pointer, 16)) return B2_E_INVALID;
    if (!is_aligned(desc->mean, 4) || !is_aligned(desc->global, 4) || !is_aligned(desc->inverse, 4)) return B2_E_INVALID;
    return b2::launch_norm_quant(desc, static_cast<cudaStream_t>(stream));
}

int b2_layer_norm_quant(const void* input, const void* update, const void* weight, const void* bias, void* residual,
                        void* output, void* scales, void* blocked, void* statistics, float scale_value, int32_t rows,
                        int32_t columns, int32_t bits, void* stream) {
    if (input == nullptr || weight == nullptr || bias == nullptr || output == nullptr || rows <= 0 || columns <= 0)
        return B2_E_INVALID;
    if (bits != 4 && bits != 8 && bits != 16) return B2_E_UNSUPPORTED;
    if (columns % 16 != 0) return B2_E_UNSUPPORTED;
    if (columns > 2048) return B2_E_TOO_LARGE;
    if (bits == 4 && blocked == nullptr) return B2_E_INVALID;
    if (bits != 16 && !(scale_value > 0.0f)) return B2_E_INVALID;
    const void* vectors[] = {input, update, weight, bias, residual, output};
    for (const void* pointer : vectors)
        if (!is_aligned(pointer, 16)) return B2_E_INVALID;
    if (!is_aligned(statistics, 4)) return B2_E_INVALID;
    return b2::launch_layer_norm_quant(input, update, weight, bias, residual, output, scales, blocked, statistics, scale_value,
                                       rows, columns, bits, static_cast<cudaStream_t>(stream));
}

int b2_bhsd_quant(const void* input, void* output, void* scales, void* blocked, float scale_value, int64_t stride_b,
                  int64_t stride_h, int64_t stride_s, int32_t batch, int32_t heads, int32_t tokens, int32_t head_dim,
                  int32_t bits, void* stream) {
    if (input == nullptr || output == nullptr || batch <= 0 || heads <= 0 || tokens <= 0 || head_dim <= 0) return B2_E_INVALID;
    if (bits != 4 && bits != 8 && bits != 16) return B2_E_UNSUPPORTED;
    if (head_dim % (bits == 4 ? 16 : 8) != 0) return B2_E_UNSUPPORTED;
    if (bits == 4 && blocked == nullptr) return B2_E_INVALID;
    if (bits != 16 && !(scale_value > 0.0f)) return B2_E_INVALID;
    if (stride_b < 0 || stride_h < 0 || stride_s < 0 || ((stride_b | stride_h | stride_s) & 7)) return B2_E_INVALID;
    if (!is_aligned(input, 16) || !is_aligned(output, 16)) return B2_E_INVALID;
    if (int64_t(batch) * tokens > 2147483647LL || int64_t(heads) * head_dim > 2147483647LL) return B2_E_TOO_LARGE;
    return b2::launch_bhsd_quant(input, output, scales, blocked, scale_value, stride_b, stride_h, stride_s, batch, heads, tokens,
                                 head_dim, bits, static_cast<cudaStream_t>(stream));
}

int b2_normalize_frames(const void* frames, void* images, int32_t cameras, int32_t pixels, void* stream) {
    if (frames == nullptr || images == nullptr || cameras <= 0 || pixels <= 0) return B2_E_INVALID;
    if (!is_aligned(images, 4)) return B2_E_INVALID;
    return b2::launch_normalize_frames(frames, images, cameras, pixels, static_cast<cudaStream_t>(stream));
}

int b2_frames_to_patches(const void* frames, void* patches, int32_t cameras, int32_t height, int32_t width, int32_t patch,
                         void* stream) {
    if (frames == nullptr || patches == nullptr || cameras <= 0 || height <= 0 || width <= 0 || patch <= 0) return B2_E_INVALID;
    if (height % patch != 0 || width % patch != 0 || (3 * patch * patch) % 4 != 0) return B2_E_UNSUPPORTED;
    if (!is_aligned(patches, 8)) return B2_E_INVALID;
    return b2::launch_frames_to_patches(frames, patches, cameras, height, width, patch, static_cast<cudaStream_t>(stream));
}

int b2_resize_frames(const void* frames, void* images, const void* row_bounds, const void* row_weights, int32_t row_taps,
                     const void* column_bounds, const void* column_weights, int32_t column_taps, int32_t cameras,
                     int32_t height, int32_t width, int32_t out_height, int32_t out_width, int32_t canvas_height,
                     int32_t canvas_width, int32_t top, int32_t left, void* stream) {
    if (frames == nullptr || images == nullptr || row_bounds == nullptr || row_weights == nullptr || column_bounds == nullptr ||
        column_weights == nullptr)
        return B2_E_INVALID;
    if (cameras <= 0 || height <= 0 || width <= 0 || out_height <= 0 || out_width <= 0 || row_taps <= 0 || column_taps <= 0)
        return B2_E_INVALID;
    if (top < 0 || left < 0 || top + out_height > canvas_height || left + out_width > canvas_width) return B2_E_INVALID;
    if (!is_aligned(images, 4) || !is_aligned(row_bounds, 4) || !is_aligned(row_weights, 4) || !is_aligned(column_bounds, 4) ||
        !is_aligned(column_weights, 4))
        return B2_E_INVALID;
    return b2::launch_resize_frames(frames, images, row_bounds, row_weights, row_taps, column_bounds, column_weights, column_taps,
                                    cameras, height, width, out_height, out_width, canvas_height, canvas_width, top, left,
                                    static_cast<cudaStream_t>(stream));
}

int64_t b2_linear_workspace_bytes(const b2_linear_desc* desc) {
    int64_t need = 0;
    if (b2::run_linear(desc, nullptr, &need) != B2_OK) return 0;
    return need;
}

}  // extern "C"
