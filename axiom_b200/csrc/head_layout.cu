// head_layout.cu — the layout passes of multi-head attention: rows of dk floats moved between the flat
// [B*S, nslot*H*dk] matrix a projection GEMM reads or writes and the head-major [B*H, S, dk] buffers the
// attention kernels use (nslot = 3 for the fused q|k|v matrix, 1 for a single tensor).  They stand behind the
// head_interleave* / head_deinterleave* slots of axiom's CUDA extension table
// (include/axiom/internal/cuda_extension.h:41-72; stock kernels src/compute/backends/cuda/ops_attention.cu:18-193).
// HBM-bound: every element is read once and written once, 128 bits at a time when dk % 4 == 0; consecutive
// threads walk the flat side, so both sides move whole dk-float rows.
#include "elementwise.cuh"

namespace axb {

struct HeadLayoutArgs {
    float *flat;        // [rows, nslot*D]
    float *head[3];     // [B*H, S, dk] per slot
    const float *bias;  // [nslot*D] or nullptr (split direction only)
    int64_t rows;       // B*S
    int nslot, S, H, dk;
    int accumulate;     // split direction only: add to what the head-major side holds instead of overwriting it
};

// TO_HEAD: flat -> head-major (+ bias); otherwise head-major -> flat.  VEC = floats per access (4 or 1).  IDX: 32-bit
// indices when every offset stays below 2^31 (four integer divisions per access: in 64 bits they, not memory, paced
// the kernel — 3.5 TB/s on the config-4 layer).
template <bool TO_HEAD, int VEC, typename IDX>
__global__ void __launch_bounds__(256) head_layout_kernel(HeadLayoutArgs a)
{
    const IDX dkv = (IDX)(a.dk / VEC);                      // accesses per head row
    const IDX H = (IDX)a.H, S = (IDX)a.S, dk = (IDX)a.dk, nslot = (IDX)a.nslot;
    const IDX D = H * dk;
    const IDX per_slot = H * dkv, per_row = nslot * per_slot;   // accesses per slot and per flat row
    const IDX total = (IDX)a.rows * per_row;
    const IDX stride = (IDX)gridDim.x * (IDX)blockDim.x;
    for (IDX i = (IDX)blockIdx.x * (IDX)blockDim.x + (IDX)threadIdx.x; i < total; i += stride) {
        const IDX row = i / per_row;
        IDX c = i - row * per_row;                          // access index inside the flat row
        const IDX which = c / per_slot;
        c -= which * per_slot;
        const IDX h = c / dkv, d = (c - h * dkv) * VEC;
        const IDX b = row / S, s = row - b * S;
        const IDX fi = row * nslot * D + which * D + h * dk + d;
        const IDX hi = ((b * H + h) * S + s) * dk + d;
        float *hp = a.head[which];
        if (VEC == 4) {
            if (TO_HEAD) {
                float4 v = *reinterpret_cast<const float4 *>(a.flat + fi);
                if (a.bias) {
                    const float4 bv = __ldg(reinterpret_cast<const float4 *>(a.bias + which * D + h * dk + d));
                    v.x += bv.x; v.y += bv.y; v.z += bv.z; v.w += bv.w;
                }
                if (a.accumulate) {
                    const float4 o = *reinterpret_cast<const float4 *>(hp + hi);
                    v.x += o.x; v.y += o.y; v.z += o.z; v.w += o.w;
                }
                *reinterpret_cast<float4 *>(hp + hi) = v;
            } else {
                *reinterpret_cast<float4 *>(a.flat + fi) = *reinterpret_cast<const float4 *>(hp + hi);
            }
        } else {
            if (TO_HEAD)
                hp[hi] = a.flat[fi] + (a.bias ? __ldg(a.bias + which * D + h * dk + d) : 0.0f) +
                         (a.accumulate ? hp[hi] : 0.0f);
            else a.flat[fi] = hp[hi];
        }
    }
}

static inline bool hl_aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

int launch_head_layout(bool to_head, float *flat, float *const head[3], const float *bias, int nslot, int64_t B,
                       int64_t S, int64_t H, int64_t dk, int sm_count, cudaStream_t st, bool accumulate)
{
    HeadLayoutArgs a;
    a.accumulate = (accumulate && to_head) ? 1 : 0;
    a.flat = flat;
    for (int i = 0; i < 3; ++i) a.head[i] = i < nslot ? head[i] : nullptr;
    a.bias = bias;
    a.rows = B * S;
    a.nslot = nslot; a.S = (int)S; a.H = (int)H; a.dk = (int)dk;
    const int64_t total = a.rows * nslot * H * dk;
    if (total <= 0) return 0;
    bool vec = (dk % 4 == 0) && hl_aligned16(flat) && (!bias || hl_aligned16(bias));
    for (int i = 0; i < nslot; ++i) vec = vec && hl_aligned16(head[i]);
    const int64_t items = vec ? total / 4 : total;
    int64_t blocks = (items + 255) / 256;
    if (blocks > (int64_t)sm_count * 16) blocks = (int64_t)sm_count * 16;
    const unsigned g = (unsigned)blocks;
    const bool narrow = total < ((int64_t)1 << 30);   // every offset and the loop index (total + grid size) inside 31 bits
#define AXB_HL_LAUNCH(TH, V)                                                          \
    do {                                                                              \
        if (narrow) head_layout_kernel<TH, V, uint32_t><<<g, 256, 0, st>>>(a);        \
        else head_layout_kernel<TH, V, int64_t><<<g, 256, 0, st>>>(a);                \
    } while (0)
    if (to_head) {
        if (vec) AXB_HL_LAUNCH(true, 4);
        else AXB_HL_LAUNCH(true, 1);
    } else {
        if (vec) AXB_HL_LAUNCH(false, 4);
        else AXB_HL_LAUNCH(false, 1);
    }
#undef AXB_HL_LAUNCH
    return (int)cudaGetLastError();
}

}  // namespace axb
