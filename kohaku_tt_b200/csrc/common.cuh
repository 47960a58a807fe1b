// Shared device helpers and the kernel-side parameter block.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/ktt_b200.h"

namespace ktt {

// The logit a masked key gets and the floor of an additive mask: finite, so a row whose
// first tiles are all masked keeps an exact fp32 running maximum
// (ktt_flash/varlen_plan.hpp:12-17).
constexpr float kMaskedLogit = -5e5f;
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

// Kernel-side view of ktt_b200_attn_args (same fields, device-friendly types).
struct AttnParams {
    int batch, heads, kv_heads, sq, sk, d, dv, causal;
    int64_t total_q, total_k;  // packed calls: rows of q and of k / v
    float scale;
    float scale_log2;  // scale * log2(e)
    const __nv_bfloat16* q;
    const __nv_bfloat16* k;
    const __nv_bfloat16* v;
    __nv_bfloat16* out;
    float* lse;
    int64_t qs[3], ks[3], vs[3], os[3], ls[3];
    const void* mask;
    int mask_dtype;
    int64_t ms[4];
    const int32_t* key_lengths;
    const int32_t* cu_q;
    const int32_t* cu_k;
    // backward
    const __nv_bfloat16* dout;
    __nv_bfloat16* dq;
    __nv_bfloat16* dk;
    __nv_bfloat16* dv_out;
    int64_t dos[3], dqs[3], dks[3], dvs[3];
    float* delta;  // [batch, heads, sq_pad] (packed: [heads, total_q_pad])
    int64_t delta_bs, delta_hs;
    // tcgen05 backward with grouped heads: the query heads of a group are split over
    // `gsplit` CTAs per key block, which leave fp32 partial dV / dK here for a reduction.
    int gsplit;
    float* dkv_partial;  // [2 (dV, dK)][batch or 1][kv_heads][gsplit][key rows x d], each 128-key block column-major in float4 units
    int32_t* fwd_work_counter;  // forward, optional: one zeroed int32 the persistent CTAs draw their items from
    int32_t* fwd_done_counter;  // with it, optional: a second zeroed int32; the kernel then leaves both zero
    int32_t* dkv_counters;  // [batch][kv_heads][key blocks] tickets of the CTAs sharing a key block; zeroed by the delta kernel
};

// One sequence's extent inside the operands.
struct SeqInfo {
    int q_off, k_off;  // packed row offsets (0 for dense)
    int lq, lk;        // rows of this batch entry
    int klen;          // keys visible by length (<= lk)
    int shift;         // causal: key j visible to query i when j <= i + shift
};

__device__ __forceinline__ SeqInfo seq_info(const AttnParams& p, int b) {
    SeqInfo s;
    if (p.cu_q) {
        s.q_off = p.cu_q[b];
        s.lq = p.cu_q[b + 1] - s.q_off;
        s.k_off = p.cu_k[b];
        s.lk = p.cu_k[b + 1] - s.k_off;
    } else {
        s.q_off = 0;
        s.k_off = 0;
        s.lq = p.sq;
        s.lk = p.sk;
    }
    s.klen = s.lk;
    if (p.key_lengths) {
        int l = p.key_lengths[b];
        l = l < 1 ? 1 : l;
        s.klen = l > s.lk ? s.lk : l;
    }
    s.shift = p.causal == KTT_B200_CAUSAL_BOTTOM_RIGHT ? s.lk - s.lq : 0;
    return s;
}

// Additive mask value (already clamped) for (b, h, query i, key j); j is the packed key
// index for packed calls.
__device__ __forceinline__ float mask_value(
    const AttnParams& p, int b, int h, int i, int64_t j) {
    const int64_t idx = b * p.ms[0] + h * p.ms[1] + i * p.ms[2] + j * p.ms[3];
    float m;
    switch (p.mask_dtype) {
        case KTT_B200_MASK_BOOL:
            return reinterpret_cast<const uint8_t*>(p.mask)[idx] ? 0.f : kMaskedLogit;
        case KTT_B200_MASK_BF16:
            m = __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p.mask)[idx]);
            break;
        case KTT_B200_MASK_F16:
            m = __half2float(reinterpret_cast<const __half*>(p.mask)[idx]);
            break;
        default:
            m = reinterpret_cast<const float*>(p.mask)[idx];
            break;
    }
    // NaN-safe clamp: -inf and anything below the floor become the masked logit.
    return m > kMaskedLogit ? m : kMaskedLogit;
}

__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));  // pure: the compiler may schedule it freely
    return y;
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 t = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&t);
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// D(16x8, f32) += A(16x16, bf16, row) * B(16x8, bf16, col)
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 "
        "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// Four transposed 8x8 b16 matrices; lane l supplies the address of one 16-byte row.
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
    asm volatile(
        "ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
        : "r"(addr));
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile(
        "ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
        : "r"(addr));
}

__device__ __forceinline__ void cp_async_16(uint32_t dst, const void* src, bool pred) {
    const int n = pred ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(n));
}
__device__ __forceinline__ void cp_async_commit() {
    asm volatile("cp.async.commit_group;\n" ::);
}
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}

// Thread-local error text and status helpers (capi.cu).
int fail(int code, const char* fmt, ...);
int check_cuda(cudaError_t e, const char* what);
// Counter slots: 0 tcgen05 forward, 1 warp-MMA forward, 2 backward, 3 decode,
// 4 refused, 5 device-wait timeouts, 6 tcgen05 backward.
void note_call(int which);

// Raises a kernel's dynamic shared-memory limit once per (kernel, device): the attribute
// is sticky, and setting it outside of every launch keeps launches legal during stream
// capture.
bool smem_limit_known(const void* kernel, int device);   // capi.cu
void smem_limit_remember(const void* kernel, int device);

template <typename K>
int ensure_smem(K kernel, int bytes, const char* what) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) dev = 0;
    const void* key = reinterpret_cast<const void*>(kernel);
    if (smem_limit_known(key, dev)) return 0;
    if (int rc = check_cuda(
            cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes), what)) {
        return rc;
    }
    smem_limit_remember(key, dev);
    return 0;
}

// Launchers (one per kernel family).
int launch_forward_mma(const AttnParams& p, cudaStream_t stream);
int launch_backward_mma(const AttnParams& p, cudaStream_t stream);
int launch_backward_delta(const AttnParams& p, cudaStream_t stream);  // delta = rowsum(dO o O)
int launch_backward_tc5(const AttnParams& p, cudaStream_t stream);
bool backward_tc5_takes(const AttnParams& p, const char** why);
// Number of CTAs the query heads of a GQA group are split over in the tcgen05 dK/dV kernel
// (1 when there are enough key blocks to fill the GPU), and the fp32 bytes that needs.
int backward_group_split(const AttnParams& p);
int64_t backward_partial_bytes(const AttnParams& p, int gsplit);
// Offset of the ticket counters inside that region (they follow the partial sums).
int64_t backward_counter_offset(const AttnParams& p, int gsplit);
int64_t backward_counter_count(const AttnParams& p, int gsplit);
int launch_forward_tc5(const AttnParams& p, cudaStream_t stream);
bool forward_tc5_takes(const AttnParams& p, const char** why);
// Head dim 64: two CTAs per SM, a thread owns a whole row of a key block (fwd_row.cu). The
// workspace (optional, forward_row_workspace() bytes, zero-filled once) holds the work
// counter and the partial results of query tiles cut in two along the keys.
bool forward_row_takes(const AttnParams& p, const char** why);
int64_t forward_row_workspace(const AttnParams& p);
int launch_forward_row(const AttnParams& p, void* workspace, int64_t workspace_bytes, cudaStream_t stream);
int forward_row_occupancy();
// 0, or KTT_B200_ERR_DEVICE_WAIT with the code of the first wait that ran out (cleared).
int device_status(int* code);
// Test support: launches one warp whose bounded wait runs out after ~1e5 cycles.
int selftest_wait_timeout(cudaStream_t stream);
// Profiling zones of the tcgen05 forward: a device buffer of 64 x 8 int64, or null.
void set_trace_buffer(long long* device_buffer);
// One query tile whose intermediate values the head-dim-64 forward writes out (ktt_b200_set_dump).
struct DumpRequest {
    float* buffer;   // device, null: no dump
    int batch, head, q_tile, max_blocks;
};
void set_dump_request(const DumpRequest& r);
DumpRequest get_dump_request();
long long* get_trace_buffer();   // what set_trace_buffer was given last, or null

}  // namespace ktt
