// Shared-memory tile movement and the score/logit rule used by the warp-MMA kernels.
#pragma once
#include "common.cuh"

namespace ktt {

constexpr int kPad = 8;  // bf16 elements of row padding: keeps fragment loads conflict-free

// Copies rows [row0, row0 + ROWS) x cols [0, dcols) of a row-major global matrix (row
// stride rs elements, nrows valid rows) into s[ROWS][DP + kPad], zero-filling the rest.
// 16-byte loads where the source chunk is whole and aligned, element loads otherwise.
template <int ROWS, int DP, int THREADS>
__device__ __forceinline__ void load_tile(
    __nv_bfloat16* s, const __nv_bfloat16* g, int64_t rs, int row0, int nrows, int dcols) {
    constexpr int CH = DP / 8;
    constexpr int LD = DP + kPad;
    for (int idx = threadIdx.x; idx < ROWS * CH; idx += THREADS) {
        const int r = idx / CH, c = idx % CH;
        uint4 val = make_uint4(0u, 0u, 0u, 0u);
        const int grow = row0 + r;
        if (grow < nrows && c * 8 < dcols) {
            const __nv_bfloat16* src = g + static_cast<int64_t>(grow) * rs + c * 8;
            if (c * 8 + 8 <= dcols && (reinterpret_cast<uintptr_t>(src) & 15) == 0) {
                val = __ldg(reinterpret_cast<const uint4*>(src));
            } else {
                __nv_bfloat16 tmp[8];
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    tmp[e] = (c * 8 + e < dcols) ? src[e] : __float2bfloat16(0.f);
                }
                val = *reinterpret_cast<uint4*>(tmp);
            }
        }
        *reinterpret_cast<uint4*>(&s[r * LD + c * 8]) = val;
    }
}

// Writes s[ROWS][DP + kPad] rows [0, ROWS) to global rows [row0, ...) (valid < nrows),
// cols [0, dcols). The caller has synchronised the writers of s.
template <int ROWS, int DP, int THREADS>
__device__ __forceinline__ void store_tile(
    const __nv_bfloat16* s, __nv_bfloat16* g, int64_t rs, int row0, int nrows, int dcols,
    int tid) {
    constexpr int CH = DP / 8;
    constexpr int LD = DP + kPad;
    for (int idx = tid; idx < ROWS * CH; idx += THREADS) {
        const int r = idx / CH, c = idx % CH;
        const int grow = row0 + r;
        if (grow < nrows && c * 8 < dcols) {
            __nv_bfloat16* dst = g + static_cast<int64_t>(grow) * rs + c * 8;
            const uint4 val = *reinterpret_cast<const uint4*>(&s[r * LD + c * 8]);
            if (c * 8 + 8 <= dcols && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
                *reinterpret_cast<uint4*>(dst) = val;
            } else {
                const __nv_bfloat16* tmp = reinterpret_cast<const __nv_bfloat16*>(&val);
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    if (c * 8 + e < dcols) dst[e] = tmp[e];
                }
            }
        }
    }
}

// Additive mask term (base 2) of (query i, key j), 0 without a mask. Indices are clamped
// into the sequence instead of tested, so the load is unconditional: the loads of a whole
// tile can then be in flight together (and ahead of the score MMAs) instead of one after
// the other behind their tests.
__device__ __forceinline__ float mask_term(const AttnParams& p, const SeqInfo& si, int b, int h, int i, int j) {
    if (p.mask_dtype == KTT_B200_MASK_NONE) return 0.f;
    const int ii = max(min(i, si.lq - 1), 0);     // rows past the end only pad the last tile
    const int jj = max(min(j, si.klen - 1), 0);
    return mask_value(p, b, h, ii, static_cast<int64_t>(si.k_off) + jj) * kLog2e;
}

// Base-2 logit of score s for (query i, key j) of sequence `si`: scale, additive mask term
// (from mask_term), key length and causal rule. -inf marks a pair that does not exist for
// this row.
__device__ __forceinline__ float logit2_with(const AttnParams& p, const SeqInfo& si, int i, int j, float s, float term) {
    const bool dead = j >= si.klen || (p.causal && j > i + si.shift);
    return dead ? -INFINITY : fmaf(s, p.scale_log2, term);
}

__device__ __forceinline__ float logit2(
    const AttnParams& p, const SeqInfo& si, int b, int h, int i, int j, float s) {
    return logit2_with(p, si, i, j, s, mask_term(p, si, b, h, i, j));
}

// A-fragment (16 rows x 16 k) of a row-major bf16 smem matrix with leading dim LD.
template <int LD>
__device__ __forceinline__ void load_a_frag(
    uint32_t (&a)[4], const __nv_bfloat16* s, int row0, int k0, int lane) {
    const int g = lane >> 2, t = lane & 3;
    const __nv_bfloat16* base = s + (row0 + g) * LD + k0 + t * 2;
    a[0] = *reinterpret_cast<const uint32_t*>(base);
    a[1] = *reinterpret_cast<const uint32_t*>(base + 8 * LD);
    a[2] = *reinterpret_cast<const uint32_t*>(base + 8);
    a[3] = *reinterpret_cast<const uint32_t*>(base + 8 * LD + 8);
}

// B-fragment (16 k x 8 n) where B[k][n] = s[n0 + n][k0 + k] (k contiguous in smem).
template <int LD>
__device__ __forceinline__ void load_b_frag(
    uint32_t& b0, uint32_t& b1, const __nv_bfloat16* s, int n0, int k0, int lane) {
    const int g = lane >> 2, t = lane & 3;
    const __nv_bfloat16* base = s + (n0 + g) * LD + k0 + t * 2;
    b0 = *reinterpret_cast<const uint32_t*>(base);
    b1 = *reinterpret_cast<const uint32_t*>(base + 8);
}

// Two B-fragments (16 k x 16 n) where B[k][n] = s[k0 + k][n0 + n] (n contiguous in
// smem): r[0], r[1] cover n0..n0+7, r[2], r[3] cover n0+8..n0+15.
template <int LD>
__device__ __forceinline__ void load_bt_frag(
    uint32_t (&r)[4], const __nv_bfloat16* s, int k0, int n0, int lane) {
    ldmatrix_x4_trans(r, smem_u32(s + (k0 + (lane & 15)) * LD + n0 + (lane >> 4) * 8));
}

}  // namespace ktt
