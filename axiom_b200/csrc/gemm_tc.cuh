// gemm_tc.cuh — interface between the tcgen05 GEMM core (gemm_tc.cu) and the
// C-ABI layer (api.cu).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace axb {

enum { TC_MAX_PLANES = 3, TC_MAX_PRODUCTS = 6, TC_MAX_EXTRA = 8 };
enum { ACT_NONE = 0, ACT_RELU = 1, ACT_GELU = 2 };
// OUT_DIGITS_T (int8 kind): the B operand is four int8 digit planes of fp32 activations, interleaved per activation row
// (B row 4*m + j = digit j of row m), the A operand the int8 weights [n][K]; accumulator row n, columns 4*m .. 4*m+3 are
// recombined with 64-bit integers by the thread that holds them and out[m][n] = act(total * colscale[n] * dg_inv_s[m] +
// bias[n]) is stored TRANSPOSED (C = out, ldc = its pitch; colscale and bias are indexed by the GEMM's row).
enum { OUT_F32 = 0, OUT_I8_REQUANT = 1, OUT_S32_ONLY = 2, OUT_DIGITS_T = 3 };

// One logical operand = up to three K-major planes [rows, k] whose sum is the
// value (a single plane for bf16 / int8; hi+lo for the split-precision modes).
struct TcOperand {
    const void *plane[TC_MAX_PLANES];
    int nplanes;
    int64_t rows;         // M for the A side, N for the B side
    int64_t pitch_elems;  // row pitch in elements (pitch * element size % 16 == 0)
};

struct TcEpilogue {
    float alpha, beta;      // f32 kinds: v = alpha * acc (* colscale[n]) (+ beta * C) (+ bias[n]) -> act
    const float *bias;      // [N] or null
    const float *colscale;  // [N] or null; int8 requant: the per-column weight scales b_scales[n]
    float rq_a_scale = 1.0f, rq_out_scale = 1.0f;   // int8 requant: out = clamp(rint(acc * ((rq_a_scale * colscale[n]) / rq_out_scale)))
    int act;                // ACT_*
    int out_mode;           // OUT_*
    void *C;                // float* (OUT_F32) / int8_t* (OUT_I8_REQUANT) / unused
    int32_t *acc_out;       // int8 kind: raw s32 accumulators, or null
    int64_t ldc;            // row pitch of C and acc_out in elements
    // fp32 kinds: further destinations that receive the same tile as C (same pitch); used to store a
    // rank's output slab straight into its peers' gather buffers over NVLink
    float *c_extra[TC_MAX_EXTRA];
    int n_extra;
    // fp32 kinds, head-major scatter (hs_dk > 0; C, ldc and c_extra are then unused, beta reads the scattered place): output column
    // which*H*dk + h*dk + d of row b*S + s goes to hs_out[which][(b*H + h)*S + s][d] — the [B*H, S, dk] layout of
    // the attention kernels.  hs_dk must be a multiple of 32 (a 32-column store never straddles two heads).
    int hs_dk = 0, hs_S = 0, hs_H = 0;
    float *hs_out[3] = { nullptr, nullptr, nullptr };
    // OUT_DIGITS_T: 2^-s of every activation row (the digits are the row's values on the grid 2^-s) and the row count
    const float *dg_inv_s = nullptr;
    int dg_rows = 0;
};

struct TcProducts {
    int n;
    int8_t a[TC_MAX_PRODUCTS], b[TC_MAX_PRODUCTS];  // plane index pairs, issued in order
    // fp32 kinds: K elements accumulated inside the tensor core before the partial
    // sum is moved to registers (0 = the whole K in one go).  The tensor core
    // truncates on accumulation, so the error of one chunk grows with its length.
    int chunk_k;
};

// Scratch the core may use to split K over several CTAs of one output tile (problems with too few tiles to fill
// the GPU).  counters must be zero on entry and are left zero.  A null pointer switches splitting off.
struct TcSplitK {
    void *scratch;
    size_t scratch_bytes;
    int *counters;
    int n_counters;
};

// Convolution as an implicit GEMM (stride 1): the B operand is not a matrix in memory but the channel-innermost
// image planes [H][W][pitch] read through shifted windows.  Output pixel (oh, ow) is row `pixel` of B; its element
// k = tap * c_pad + c (tap = ky * kw + kx) is image[oh + ky - pad_h][ow + kx - pad_w][c], zero outside the image
// and for c >= C — each pipeline stage is one TMA box per 64-pixel patch at window-shifted coordinates, and the
// zero fill of out-of-range coordinates IS the padding.  The A operand (the filter) is laid out to match:
// [M][taps * c_pad] with c_pad = C rounded up to gemm_tc_conv_channel_pad(kind).  The output [batch][M][out_h][out_w] is
// written in 16-byte groups that must not straddle pixel rows, so out_w % 4 == 0 and a 16-byte aligned base are
// required (gemm_tc_conv_applicable).
struct TcConv {
    int64_t C, H, W;       // image planes: C valid channels per pixel (B.pitch_elems apart)
    int kh, kw, pad_h, pad_w;
    int64_t out_h, out_w;
    int64_t batch = 1;     // samples: image planes [batch][H][W][pitch], output [batch][M][out_h][out_w]
};
int gemm_tc_conv_channel_pad(int kind);
bool gemm_tc_conv_applicable(const TcConv &cv, int sh, int sw, const void *out);
// ep.C = out [M][out_h][out_w] fp32; alpha and act are applied, beta must be 0, no bias, no extra destinations
int launch_gemm_tc_conv(int kind, const TcOperand &A, const TcOperand &B_image, const TcProducts &prod, int64_t M,
                        const TcConv &cv, const TcEpilogue &ep, int *err_word, int sm_count, cudaStream_t stream,
                        const TcSplitK *splitk = nullptr);

// kind: MmaKind (0 tf32, 1 bf16, 2 int8).  Returns cudaError_t as int; a device
// side wait that ran out is reported through *err_word (0 = clean).
int launch_gemm_tc(int kind, const TcOperand &A, const TcOperand &B, const TcProducts &prod,
                   int64_t M, int64_t N, int64_t K, const TcEpilogue &ep, int *err_word,
                   int sm_count, cudaStream_t stream, const TcSplitK *splitk = nullptr);

// Whether launch_gemm_tc would cut K into slices for this problem when given scratch: callers that multiply row
// blocks of one problem in separate launches ask, because a split changes the order of the fp32 additions.
bool gemm_tc_splits_k(int kind, const TcProducts &prod, int64_t M, int64_t N, int64_t K, int sm_count);

// Message of the last failure in this translation unit (tensor-map encoding, launch).
const char *gemm_tc_last_error();

// Tiled tensor map (128 bytes, 64-byte aligned storage at tmap_out) over a plain
// fp32 matrix [rows, cols] with row pitch pitch_elems; no swizzle; out-of-range
// elements read as zero.  pitch_elems * 4 and the base must be multiples of 16 bytes.
int encode_f32_matrix_tmap(void *tmap_out, const float *ptr, int64_t rows, int64_t cols, int64_t pitch_elems,
                           int box_cols, int box_rows);

// Tiled tensor map over fp32 planes [batch][rows][pitch_elems] (cols valid elements per row), 128-byte swizzle,
// box = 32 elements x box_rows x 1; out-of-range rows / columns read as zero.  atom32 selects the variant of
// the swizzle that moves 32-byte chunks (for MN-major tf32 MMA operands).
int encode_f32_batched_tmap(void *tmap_out, const void *ptr, int64_t batch, int64_t rows, int64_t cols,
                            int64_t pitch_elems, int box_rows, bool atom32);
// int8 planes [batch][rows][pitch_bytes], 128-byte swizzle, box = 128 bytes x box_rows x box_batch; out-of-range reads are zero
int encode_i8_batched_tmap(void *tmap_out, const void *ptr, int64_t batch, int64_t rows, int64_t cols,
                           int64_t pitch_bytes, int64_t batch_stride_bytes, int box_rows, int box_batch);

}  // namespace axb
