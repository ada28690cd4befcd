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

// TO_HEAD: flat -> head-major (+ bias); otherwise head-major -> flat.  VEC = floats per access (4 or 1).
template <bool TO_HEAD, int VEC>
__global__ void __launch_bounds__(256) head_layout_kernel(HeadLayoutArgs a)
{
    const int dkv = a.dk / VEC;                             // accesses per head row
    const int64_t D = (int64_t)a.H * a.dk;
    const int64_t per_row = (int64_t)a.nslot * a.H * dkv;   // accesses per flat row
    const int64_t total = a.rows * per_row;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t row = i / per_row;
        int64_t c = i - row * per_row;                      // access index inside the flat row
        const int which = (int)(c / ((int64_t)a.H * dkv));
        c -= (int64_t)which * a.H * dkv;
        const int h = (int)(c / dkv), d = (int)(c - (int64_t)h * dkv) * VEC;
        const int64_t b = row / a.S, s = row - b * a.S;
        const int64_t fi = row * a.nslot * D + (int64_t)which * D + (int64_t)h * a.dk + d;
        const int64_t hi = ((b * a.H + h) * a.S + s) * a.dk + d;
        float *hp = a.head[which];
        if (VEC == 4) {
            if (TO_HEAD) {
                float4 v = *reinterpret_cast<const float4 *>(a.flat + fi);
                if (a.bias) {
                    const float4 bv = __ldg(reinterpret_cast<const float4 *>(a.bias + (int64_t)which * D + (int64_t)h * a.dk + d));
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
                hp[hi] = a.flat[fi] + (a.bias ? __ldg(a.bias + (int64_t)which * D + (int64_t)h * a.dk + d) : 0.0f) +
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
    if (to_head) {
        if (vec) head_layout_kernel<true, 4><<<g, 256, 0, st>>>(a);
        else head_layout_kernel<true, 1><<<g, 256, 0, st>>>(a);
    } else {
        if (vec) head_layout_kernel<false, 4><<<g, 256, 0, st>>>(a);
        else head_layout_kernel<false, 1><<<g, 256, 0, st>>>(a);
    }
    return (int)cudaGetLastError();
}

}  // namespace axb
