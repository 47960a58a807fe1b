// The extern "C" surface: argument checks, kernel choice, counters, error text.
#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <set>
#include <utility>

#include "common.cuh"

namespace ktt {

namespace {
thread_local char g_error[512] = "";
std::atomic<int64_t> g_counters[8];
}  // namespace

int fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
    return code;
}

int check_cuda(cudaError_t e, const char* what) {
    if (e == cudaSuccess) return 0;
    return fail(KTT_B200_ERR_LAUNCH, "%s: %s", what, cudaGetErrorString(e));
}

void note_call(int which) { g_counters[which].fetch_add(1, std::memory_order_relaxed); }

namespace {
std::mutex g_smem_mutex;
std::set<std::pair<const void*, int>> g_smem_done;
}  // namespace

bool smem_limit_known(const void* kernel, int device) {
    std::lock_guard<std::mutex> lock(g_smem_mutex);
    return g_smem_done.count({kernel, device}) != 0;
}

void smem_limit_remember(const void* kernel, int device) {
    std::lock_guard<std::mutex> lock(g_smem_mutex);
    g_smem_done.insert({kernel, device});
}

namespace {

// The first condition a forward call fails, or null. Mirrors the shape rules of
// fused_refusal (aten_attention.cpp:62-127) and ktt_flash::refusal
// (ktt_flash/program.cpp:847-910) that still mean something on this hardware.
const char* forward_refusal(const ktt_b200_attn_args* a) {
    if (!a) return "null arguments";
    if (a->batch < 1 || a->heads < 1 || a->kv_heads < 1 || a->sq < 1 || a->sk < 1 || a->d < 1 || a->dv < 1) {
        return "q, k and v must be non-empty";
    }
    if (a->heads % a->kv_heads) return "q, k and v shapes do not match (K / V heads must divide Q heads)";
    if (a->d > 256 || a->dv > 256) return "head dims above 256 are not taken";
    if (a->batch > 65535 || a->heads > 65535) return "batch and heads must not exceed 65535";
    if (a->causal < 0 || a->causal > 2) return "unknown causal mode";
    if (a->causal && a->mask_dtype != KTT_B200_MASK_NONE && !a->cu_seqlens_q) return "causal takes no mask";
    if (a->mask_dtype < 0 || a->mask_dtype > KTT_B200_MASK_F16) return "unknown mask dtype";
    if ((a->mask_dtype != KTT_B200_MASK_NONE) != (a->mask != nullptr)) return "mask pointer and mask dtype disagree";
    if ((a->cu_seqlens_q == nullptr) != (a->cu_seqlens_k == nullptr)) return "packed calls need both offset arrays";
    if (a->cu_seqlens_q && a->causal == KTT_B200_CAUSAL_TOP_LEFT) return "packed causal attention is bottom-right aligned";
    if (a->cu_seqlens_q && a->key_lengths) return "packed calls take no key lengths";
    if (!(a->scale == a->scale) || a->scale <= 0.f) return "the softmax scale must be positive";
    return nullptr;
}

const char* backward_refusal(const ktt_b200_attn_args* a) {
    if (const char* why = forward_refusal(a)) return why;
    return nullptr;
}

void to_params(const ktt_b200_attn_args* a, AttnParams& p) {
    std::memset(&p, 0, sizeof(p));
    p.batch = a->batch; p.heads = a->heads; p.kv_heads = a->kv_heads;
    p.sq = a->sq; p.sk = a->sk; p.d = a->d; p.dv = a->dv; p.causal = a->causal;
    p.total_q = a->total_q; p.total_k = a->total_k;
    p.scale = a->scale;
    p.scale_log2 = a->scale * kLog2e;
    p.q = static_cast<const __nv_bfloat16*>(a->q);
    p.k = static_cast<const __nv_bfloat16*>(a->k);
    p.v = static_cast<const __nv_bfloat16*>(a->v);
    p.out = static_cast<__nv_bfloat16*>(a->out);
    p.lse = a->lse;
    for (int i = 0; i < 3; ++i) {
        p.qs[i] = a->q_strides[i]; p.ks[i] = a->k_strides[i]; p.vs[i] = a->v_strides[i];
        p.os[i] = a->out_strides[i]; p.ls[i] = a->lse_strides[i];
        p.dos[i] = a->dout_strides[i]; p.dqs[i] = a->dq_strides[i];
        p.dks[i] = a->dk_strides[i]; p.dvs[i] = a->dv_strides[i];
    }
    p.mask = a->mask;
    p.mask_dtype = a->mask_dtype;
    for (int i = 0; i < 4; ++i) p.ms[i] = a->mask_strides[i];
    p.key_lengths = a->key_lengths;
    p.cu_q = a->cu_seqlens_q;
    p.cu_k = a->cu_seqlens_k;
    p.dout = static_cast<const __nv_bfloat16*>(a->dout);
    p.dq = static_cast<__nv_bfloat16*>(a->dq);
    p.dk = static_cast<__nv_bfloat16*>(a->dk);
    p.dv_out = static_cast<__nv_bfloat16*>(a->dv_out);
}

// Rows of the delta workspace: one fp32 per (batch, head, query row).
void delta_layout(const ktt_b200_attn_args* a, int64_t& bs, int64_t& hs, int64_t& total) {
    if (a->cu_seqlens_q) {
        hs = (a->total_q + 63) / 64 * 64;
        bs = 0;
        total = hs * a->heads;
    } else {
        hs = (static_cast<int64_t>(a->sq) + 63) / 64 * 64;
        bs = hs * a->heads;
        total = bs * a->batch;
    }
}

__global__ void merge_partials_kernel(
    void* out, float* lse, const void* out2, const float* lse2, int64_t rows, int dv, int f32, int vec) {
    const int64_t row = blockIdx.x * static_cast<int64_t>(blockDim.y) + threadIdx.y;
    if (row >= rows) return;
    const float a = lse[row], b = lse2[row];
    const float m = fmaxf(a, b);
    float wa, wb, l;
    if (m == -INFINITY) {
        wa = 0.f; wb = 0.f; l = -INFINITY;
    } else {
        const float ea = __expf(a - m), eb = __expf(b - m);
        wa = ea / (ea + eb);
        wb = eb / (ea + eb);
        l = m + __logf(ea + eb);
    }
    // f32: 0 = both bf16, 1 = both fp32, 2 = fp32 accumulator with a bf16 second operand.
    if (vec) {
        for (int c = threadIdx.x * 4; c < dv; c += blockDim.x * 4) {
            const int64_t i = row * dv + c;
            float x[4], y[4];
            if (f32) {
                const float4 t = *reinterpret_cast<const float4*>(static_cast<const float*>(out) + i);
                x[0] = t.x; x[1] = t.y; x[2] = t.z; x[3] = t.w;
            } else {
                const uint2 t = *reinterpret_cast<const uint2*>(static_cast<const __nv_bfloat16*>(out) + i);
                const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&t.x));
                const float2 hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&t.y));
                x[0] = lo.x; x[1] = lo.y; x[2] = hi.x; x[3] = hi.y;
            }
            if (f32 == 1) {
                const float4 t = *reinterpret_cast<const float4*>(static_cast<const float*>(out2) + i);
                y[0] = t.x; y[1] = t.y; y[2] = t.z; y[3] = t.w;
            } else {
                const uint2 t = *reinterpret_cast<const uint2*>(static_cast<const __nv_bfloat16*>(out2) + i);
                const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&t.x));
                const float2 hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&t.y));
                y[0] = lo.x; y[1] = lo.y; y[2] = hi.x; y[3] = hi.y;
            }
#pragma unroll
            for (int e = 0; e < 4; ++e) x[e] = x[e] * wa + y[e] * wb;
            if (f32) {
                *reinterpret_cast<float4*>(static_cast<float*>(out) + i) = make_float4(x[0], x[1], x[2], x[3]);
            } else {
                uint2 t;
                t.x = pack_bf16(x[0], x[1]);
                t.y = pack_bf16(x[2], x[3]);
                *reinterpret_cast<uint2*>(static_cast<__nv_bfloat16*>(out) + i) = t;
            }
        }
    } else {
        for (int c = threadIdx.x; c < dv; c += blockDim.x) {
            const int64_t i = row * dv + c;
            const float y = f32 == 1 ? static_cast<const float*>(out2)[i]
                                     : __bfloat162float(static_cast<const __nv_bfloat16*>(out2)[i]);
            if (f32) {
                float* o = static_cast<float*>(out);
                o[i] = o[i] * wa + y * wb;
            } else {
                __nv_bfloat16* o = static_cast<__nv_bfloat16*>(out);
                o[i] = __float2bfloat16(__bfloat162float(o[i]) * wa + y * wb);
            }
        }
    }
    __syncwarp();  // one warp per row: every lane has read lse[row]
    if (threadIdx.x == 0) lse[row] = l;
}

}  // namespace
}  // namespace ktt

using namespace ktt;

extern "C" int ktt_b200_abi_version(void) { return KTT_B200_ABI_VERSION; }

extern "C" const char* ktt_b200_last_error(void) { return g_error; }

extern "C" int ktt_b200_counters(int64_t* out8) {
    if (!out8) return fail(KTT_B200_ERR_BAD_ARGUMENT, "counters: null output");
    for (int i = 0; i < 8; ++i) out8[i] = g_counters[i].load(std::memory_order_relaxed);
    return 0;
}

extern "C" int ktt_b200_device_status(int* code) {
    int c = 0;
    const int rc = device_status(&c);
    if (code) *code = c;
    if (rc) return fail(rc, "a tcgen05 kernel gave up waiting (code %d)", c);
    return 0;
}

__global__ void __launch_bounds__(256) probe_read_kernel(const uint4* data, int64_t vectors, int32_t* sink) {
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    uint32_t acc = 0;
    int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    // Four independent loads in flight per thread.
    for (; i + 3 * stride < vectors; i += 4 * stride) {
        const uint4 a = __ldcs(data + i), b = __ldcs(data + i + stride), c = __ldcs(data + i + 2 * stride),
                    d = __ldcs(data + i + 3 * stride);
        acc ^= a.x ^ a.y ^ a.z ^ a.w ^ b.x ^ b.y ^ b.z ^ b.w ^ c.x ^ c.y ^ c.z ^ c.w ^ d.x ^ d.y ^ d.z ^ d.w;
    }
    for (; i < vectors; i += stride) {
        const uint4 a = __ldcs(data + i);
        acc ^= a.x ^ a.y ^ a.z ^ a.w;
    }
    if (acc == 0x9e3779b9u) *sink = 1;   // practically never: keeps the loads alive
}

extern "C" int ktt_b200_probe_read(const void* data, int64_t bytes, int32_t* sink, void* stream) {
    if (!data || !sink || bytes < 0 || (bytes & 15) || (reinterpret_cast<uintptr_t>(data) & 15)) {
        return fail(KTT_B200_ERR_BAD_ARGUMENT, "probe_read: a 16-byte aligned buffer of a multiple of 16 bytes and a sink are needed");
    }
    if (bytes == 0) return 0;
    int dev = 0, sms = 148;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    probe_read_kernel<<<2 * sms, 256, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<const uint4*>(data), bytes / 16, sink);
    return check_cuda(cudaGetLastError(), "probe_read launch");
}

extern "C" int ktt_b200_selftest_wait_timeout(void* stream) {
    return selftest_wait_timeout(static_cast<cudaStream_t>(stream));
}

extern "C" int ktt_b200_set_dump(float* device_buffer, int32_t batch, int32_t head, int32_t q_tile, int32_t max_blocks) {
    if (device_buffer && (batch < 0 || head < 0 || q_tile < 0 || max_blocks < 1)) {
        return fail(KTT_B200_ERR_BAD_ARGUMENT, "set_dump: negative index or no room for a key block");
    }
    DumpRequest r;
    r.buffer = device_buffer;
    r.batch = batch;
    r.head = head;
    r.q_tile = q_tile;
    r.max_blocks = max_blocks;
    set_dump_request(r);
    return 0;
}

extern "C" int ktt_b200_set_trace(void* device_buffer) {
    set_trace_buffer(static_cast<long long*>(device_buffer));
    return 0;
}

extern "C" int ktt_b200_reset_counters(void) {
    for (auto& c : g_counters) c.store(0, std::memory_order_relaxed);
    return 0;
}

extern "C" int ktt_b200_sdpa_supported(const ktt_b200_attn_args* a) {
    if (const char* why = forward_refusal(a)) {
        fail(KTT_B200_ERR_UNSUPPORTED, "%s", why);
        return 0;
    }
    if (a->kernel == KTT_B200_KERNEL_TC5 || a->kernel == KTT_B200_KERNEL_TC5_WIDE) {
        AttnParams p;
        to_params(a, p);
        const char* why = nullptr;
        if (!forward_tc5_takes(p, &why)) {
            fail(KTT_B200_ERR_UNSUPPORTED, "tcgen05 kernel: %s", why);
            return 0;
        }
    }
    return 1;
}

extern "C" int ktt_b200_sdpa_backward_supported(const ktt_b200_attn_args* a) {
    if (const char* why = backward_refusal(a)) {
        fail(KTT_B200_ERR_UNSUPPORTED, "%s", why);
        return 0;
    }
    return 1;
}

extern "C" int ktt_b200_sdpa_forward(const ktt_b200_attn_args* a, void* stream) {
    if (const char* why = forward_refusal(a)) {
        note_call(4);
        return fail(KTT_B200_ERR_UNSUPPORTED, "sdpa_forward: %s", why);
    }
    if (!a->q || !a->k || !a->v || !a->out) {
        return fail(KTT_B200_ERR_BAD_ARGUMENT, "sdpa_forward: null tensor pointer");
    }
    AttnParams p;
    to_params(a, p);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const char* why = nullptr;
    const bool tc5 = forward_tc5_takes(p, &why);
    const bool wants_tc5 = a->kernel == KTT_B200_KERNEL_TC5 || a->kernel == KTT_B200_KERNEL_TC5_WIDE;
    if (wants_tc5 && !tc5) {
        note_call(4);
        return fail(KTT_B200_ERR_UNSUPPORTED, "sdpa_forward: tcgen05 kernel: %s", why);
    }
    if (tc5 && a->kernel != KTT_B200_KERNEL_MMA) {
        note_call(0);
        const char* why_row = nullptr;
        if (a->kernel != KTT_B200_KERNEL_TC5_WIDE && forward_row_takes(p, &why_row)) {
            return launch_forward_row(p, a->workspace, a->workspace_bytes, st);
        }
        // The one-CTA-per-SM kernel draws its items from a counter in the workspace: with the
        // full workspace (ktt_b200_sdpa_forward_workspace bytes) it puts the counter back to
        // zero itself; a 4..255-byte workspace is one int32 the caller zeroes before every call.
        const bool usable = a->workspace && (reinterpret_cast<uintptr_t>(a->workspace) & 3) == 0;
        p.fwd_work_counter = (usable && a->workspace_bytes >= 4) ? static_cast<int32_t*>(a->workspace) : nullptr;
        p.fwd_done_counter = (usable && a->workspace_bytes >= 256) ? static_cast<int32_t*>(a->workspace) + 1 : nullptr;
        return launch_forward_tc5(p, st);
    }
    note_call(1);
    return launch_forward_mma(p, st);
}

extern "C" int64_t ktt_b200_sdpa_forward_workspace(const ktt_b200_attn_args* a) {
    if (const char* why = forward_refusal(a)) {
        fail(KTT_B200_ERR_UNSUPPORTED, "%s", why);
        return 0;
    }
    if (a->kernel == KTT_B200_KERNEL_MMA) return 0;
    AttnParams p;
    to_params(a, p);
    const char* why = nullptr;
    if (!forward_tc5_takes(p, &why)) return 0;   // the warp-MMA kernel has no use for one
    return forward_row_workspace(p);             // the same 256 bytes for both tcgen05 kernels
}

extern "C" int ktt_b200_forward_streams_per_sm(void) { return forward_row_occupancy(); }

extern "C" int64_t ktt_b200_sdpa_backward_workspace(const ktt_b200_attn_args* a) {
    if (const char* why = backward_refusal(a)) {
        fail(KTT_B200_ERR_UNSUPPORTED, "%s", why);
        return 0;
    }
    int64_t bs, hs, total;
    delta_layout(a, bs, hs, total);
    AttnParams p;
    to_params(a, p);
    return (total * 4 + 255) / 256 * 256 + backward_partial_bytes(p, backward_group_split(p));
}

// Packed calls: rows of dq, dk and dv that no sequence of the offsets covers (before the
// first offset, after the last) get zeros here; every row inside a sequence is written by the
// CTA that owns it, so callers need not clear the gradients first.
__global__ void zero_uncovered_rows_kernel(const AttnParams p) {
    const int64_t q_lo = p.cu_q[0], q_hi = p.cu_q[p.batch], k_lo = p.cu_k[0], k_hi = p.cu_k[p.batch];
    const int64_t q_rows = q_lo + (p.total_q - q_hi), k_rows = k_lo + (p.total_k - k_hi);
    if (q_rows <= 0 && k_rows <= 0) return;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x, t0 = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    const __nv_bfloat16 zero = __float2bfloat16(0.f);
    auto clear = [&](__nv_bfloat16* base, const int64_t (&st)[3], int heads, int d, int64_t lo, int64_t hi, int64_t total) {
        const int64_t rows = lo + (total - hi);
        for (int64_t i = t0; i < rows * heads * d; i += stride) {
            const int e = static_cast<int>(i % d);
            const int h = static_cast<int>((i / d) % heads);
            const int64_t r = i / (static_cast<int64_t>(d) * heads);
            const int64_t row = r < lo ? r : hi + (r - lo);
            base[h * st[1] + row * st[2] + e] = zero;
        }
    };
    clear(p.dq, p.dqs, p.heads, p.d, q_lo, q_hi, p.total_q);
    clear(p.dk, p.dks, p.kv_heads, p.d, k_lo, k_hi, p.total_k);
    clear(p.dv_out, p.dvs, p.kv_heads, p.dv, k_lo, k_hi, p.total_k);
}

extern "C" int ktt_b200_sdpa_backward(const ktt_b200_attn_args* a, void* stream) {
    if (const char* why = backward_refusal(a)) {
        note_call(4);
        return fail(KTT_B200_ERR_UNSUPPORTED, "sdpa_backward: %s", why);
    }
    if (!a->q || !a->k || !a->v || !a->out || !a->lse || !a->dout || !a->dq || !a->dk || !a->dv_out) {
        return fail(KTT_B200_ERR_BAD_ARGUMENT, "sdpa_backward: null tensor pointer");
    }
    int64_t bs, hs, total;
    delta_layout(a, bs, hs, total);
    AttnParams p;
    to_params(a, p);
    const int64_t delta_bytes = (total * 4 + 255) / 256 * 256;
    p.gsplit = backward_group_split(p);
    const int64_t need = delta_bytes + backward_partial_bytes(p, p.gsplit);
    if (!a->workspace || a->workspace_bytes < need) {
        return fail(KTT_B200_ERR_BAD_ARGUMENT, "sdpa_backward: workspace holds %lld bytes, %lld needed",
                    static_cast<long long>(a->workspace_bytes), static_cast<long long>(need));
    }
    p.delta = static_cast<float*>(a->workspace);
    p.delta_bs = bs;
    p.delta_hs = hs;
    p.dkv_partial = reinterpret_cast<float*>(static_cast<unsigned char*>(a->workspace) + delta_bytes);
    p.dkv_counters = p.gsplit > 1
        ? reinterpret_cast<int32_t*>(static_cast<unsigned char*>(a->workspace) + delta_bytes + backward_counter_offset(p, p.gsplit))
        : nullptr;
    note_call(2);
    if (p.cu_q) {
        zero_uncovered_rows_kernel<<<64, 256, 0, static_cast<cudaStream_t>(stream)>>>(p);
        if (int rc = check_cuda(cudaGetLastError(), "zero_uncovered_rows launch")) return rc;
    }
    const char* why = nullptr;
    const bool tc5 = backward_tc5_takes(p, &why);
    if (a->kernel == KTT_B200_KERNEL_TC5 && !tc5) {
        note_call(4);
        return fail(KTT_B200_ERR_UNSUPPORTED, "sdpa_backward: tcgen05 kernel: %s", why);
    }
    if (tc5 && a->kernel != KTT_B200_KERNEL_MMA) {
        note_call(6);
        return launch_backward_tc5(p, static_cast<cudaStream_t>(stream));
    }
    return launch_backward_mma(p, static_cast<cudaStream_t>(stream));
}

extern "C" int ktt_b200_merge_partials(
    void* out, float* lse, const void* out2, const float* lse2,
    int64_t rows, int32_t dv, int32_t out_is_f32, void* stream) {
    if (!out || !lse || !out2 || !lse2 || rows < 0 || dv < 1) {
        return fail(KTT_B200_ERR_BAD_ARGUMENT, "merge_partials: null pointer or bad size");
    }
    if (out_is_f32 < 0 || out_is_f32 > 2) return fail(KTT_B200_ERR_BAD_ARGUMENT, "merge_partials: out_is_f32 must be 0, 1 or 2");
    if (rows == 0) return 0;
    dim3 block(32, 8);
    const int64_t blocks = (rows + 7) / 8;
    // Four values per access only where both operands allow it: rows of a multiple of four
    // values whose first element is 16-byte (fp32) or 8-byte (bf16) aligned.
    const uintptr_t need_out = out_is_f32 ? 15 : 7, need_out2 = out_is_f32 == 1 ? 15 : 7;
    const int vec = (dv & 3) == 0 && (reinterpret_cast<uintptr_t>(out) & need_out) == 0 &&
                    (reinterpret_cast<uintptr_t>(out2) & need_out2) == 0;
    merge_partials_kernel<<<static_cast<unsigned>(blocks), block, 0, static_cast<cudaStream_t>(stream)>>>(
        out, lse, out2, lse2, rows, dv, out_is_f32, vec);
    return check_cuda(cudaGetLastError(), "merge_partials launch");
}
