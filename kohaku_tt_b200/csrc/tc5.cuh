// Shared pieces of the TMA + tcgen05 kernels: PTX wrappers, descriptors, the bounded
// mbarrier wait, and the host-side tensor-map helpers.
#pragma once
#include <cuda.h>

#include "common.cuh"

namespace ktt {
namespace tc5 {

constexpr int kBM = 128;          // rows of the stationary operand tile per CTA (MMA M)
constexpr int kBN = 128;          // rows of the streamed operand per block (MMA N of the score MMA)
constexpr long long kWaitCycles = 4000000000ll;  // about two seconds

// ---- PTX wrappers ---------------------------------------------------------------------

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {  // one elected lane
    asm volatile(
        "{\n.reg .pred q;\n"
        "elect.sync _|q, 0xffffffff;\n"
        "@q mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n}"
        ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// One arrival for the whole (converged) warp: the lanes meet, lane 0 arrives. The barrier
// counts warps, not threads, so a phase costs a handful of shared-memory updates instead of
// one per thread.
__device__ __forceinline__ void mbar_arrive_warp(uint32_t bar) {
    __syncwarp();
    if ((threadIdx.x & 31) == 0) mbar_arrive(bar);
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n.reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.b32 %0, 1, 0, p;\n}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}

// Division by a number fixed at launch, for 0 <= n < 2^31: a multiply and a shift where the
// integer division of a runtime value is a chain of some twenty dependent instructions. A
// kernel that finds its tile from an index does several of them one after the other, with
// nothing to overlap.
struct Divisor {
    uint32_t mul, shift, d;
};
inline Divisor divisor_of(int d) {
    Divisor f;
    f.d = static_cast<uint32_t>(d);
    f.shift = 0;
    while ((1u << f.shift) < f.d) ++f.shift;   // ceil(log2 d)
    f.mul = static_cast<uint32_t>(((1ull << 32) * ((1ull << f.shift) - f.d)) / f.d + 1);
    return f;
}
__device__ __forceinline__ int div_by(int n, const Divisor& f) {
    return static_cast<int>((__umulhi(static_cast<uint32_t>(n), f.mul) + static_cast<uint32_t>(n)) >> f.shift);
}
__device__ __forceinline__ int mod_by(int n, const Divisor& f) {
    return n - div_by(n, f) * static_cast<int>(f.d);
}

// Sixteen bf16 values (eight packed words) to global memory: one 32-byte store where the
// address allows it, else two 16-byte ones. A thread that owns a row of a tile writes into a
// line of its own, so the load/store unit's time on the tile goes with the number of store
// instructions, not with their width.
__device__ __forceinline__ void store_32_bytes(void* dst, const uint32_t (&w)[8]) {
    if ((reinterpret_cast<uintptr_t>(dst) & 31) == 0) {
        asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
                     ::"l"(dst), "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3]), "r"(w[4]), "r"(w[5]), "r"(w[6]), "r"(w[7]) : "memory");
    } else {
        reinterpret_cast<uint4*>(dst)[0] = make_uint4(w[0], w[1], w[2], w[3]);
        reinterpret_cast<uint4*>(dst)[1] = make_uint4(w[4], w[5], w[6], w[7]);
    }
}

// Bounded wait. Returns false when it gave up (its own limit, or another role's).
__device__ __noinline__ inline bool mbar_wait_slow(
    uint32_t bar, uint32_t parity, volatile int* abort_flag, int code, int* status, long long limit = kWaitCycles) {
    const long long t0 = clock64();
    while (true) {
        if (mbar_try_wait(bar, parity)) return true;
        if (*abort_flag) return false;
        if (clock64() - t0 > limit) {
            *abort_flag = 1;
            atomicCAS_system(status, 0, code);
            return false;
        }
    }
}
__device__ __forceinline__ bool mbar_wait(
    uint32_t bar, uint32_t parity, volatile int* abort_flag, int code, int* status) {
    if (mbar_try_wait(bar, parity)) return true;
    return mbar_wait_slow(bar, parity, abort_flag, code, status);
}

__device__ __forceinline__ void tma_load_4d(
    uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1, int c2, int c3) {
    asm volatile(  // one elected lane of the converged producer warp
        "{\n.reg .pred q;\n"
        "elect.sync _|q, 0xffffffff;\n"
        "@q cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
        "[%0], [%1, {%3, %4, %5, %6}], [%2];\n}"
        ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
        : "memory");
}

__device__ __forceinline__ void tmem_alloc(uint32_t smem_dst, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void fence_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
// The tensor-core and TMA instructions below are issued by one elected lane of a CONVERGED
// warp: every lane of the role's warp executes the surrounding code and `elect.sync`
// predicates the instruction itself. Measured on B200: the same tcgen05.mma issued from a
// lone lane of a diverged warp (the other lanes parked at a barrier) takes ~265 cycles per
// instruction whatever its shape; from a converged warp it runs at the tensor core's rate
// (65 cycles for 128 x 128 x 16).
__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile(
        "{\n.reg .pred q;\n"
        "elect.sync _|q, 0xffffffff;\n"
        "@q tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n}"
        ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_mma(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n.reg .pred p, q;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "elect.sync _|q, 0xffffffff;\n"
        "@q tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}"
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// Same with the A operand in tensor memory (P): [a_tmem] holds 128 lanes x 8 columns of
// packed bf16 pairs per K = 16 step.
__device__ __forceinline__ void tc_mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n.reg .pred p, q;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "elect.sync _|q, 0xffffffff;\n"
        "@q tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// 16 consecutive 32-bit columns of this thread's TMEM lane (32 packed bf16 values).
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t* r) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%16], "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15};"
        ::"r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
          "r"(taddr)
        : "memory");
}

// 8 consecutive 32-bit columns of this thread's TMEM lane (16 packed bf16 values).
__device__ __forceinline__ void tmem_st8(uint32_t taddr, const uint32_t* r) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x8.b32 [%8], {%0, %1, %2, %3, %4, %5, %6, %7};"
        ::"r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(taddr)
        : "memory");
}

// 32 consecutive fp32 columns of this thread's TMEM lane.
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float* v) {
    uint32_t* r = reinterpret_cast<uint32_t*>(v);
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
// 16 consecutive fp32 columns of this thread's TMEM lane.
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, float* v) {
    uint32_t* r = reinterpret_cast<uint32_t*>(v);
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const float* v) {
    const uint32_t* r = reinterpret_cast<const uint32_t*>(v);
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%32], "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31};"
        ::"r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
          "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
          "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31]),
          "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// 2^x on the FMA pipe: round-to-nearest split x = n + f with the 1.5 * 2^23 trick, a cubic
// for 2^f on [-0.5, 0.5] (max relative error 7.5e-5, far inside bf16 rounding) and n added
// to the exponent field. The reference evaluates its exponentials the same way, with a
// degree-2 polynomial on the multiply-add path (ktt_flash/sfpu.hpp:29-30).
__device__ __forceinline__ float exp2_poly(float x) {
    x = fmaxf(x, -125.f);
    const float t = x + 12582912.f;
    const float f = x - (t - 12582912.f);
    float r = fmaf(f, 0.0551716648f, 0.2426111251f);
    r = fmaf(r, f, 0.6932609677f);
    r = fmaf(r, f, 0.9999280572f);
    return __int_as_float(__float_as_int(r) + (__float_as_int(t) << 23));
}

// The same for two values at once on the packed fp32 pipe (fma.rn.f32x2 / add.f32x2 halve
// the instruction count of the softmax loop, which is issue-bound).
__device__ __forceinline__ float2 exp2_poly2(float2 x) {
    const float2 magic = make_float2(12582912.f, 12582912.f);
    x.x = fmaxf(x.x, -125.f);
    x.y = fmaxf(x.y, -125.f);
    const float2 t = __fadd2_rn(x, magic);
    const float2 n = __fadd2_rn(t, make_float2(-12582912.f, -12582912.f));
    const float2 f = __ffma2_rn(n, make_float2(-1.f, -1.f), x);
    float2 r = __ffma2_rn(f, make_float2(0.0551716648f, 0.0551716648f), make_float2(0.2426111251f, 0.2426111251f));
    r = __ffma2_rn(r, f, make_float2(0.6932609677f, 0.6932609677f));
    r = __ffma2_rn(r, f, make_float2(0.9999280572f, 0.9999280572f));
    // n into the exponent field: one integer multiply-add per value (wraps like a shift).
    r.x = __int_as_float(__float_as_int(t.x) * (1 << 23) + __float_as_int(r.x));
    r.y = __int_as_float(__float_as_int(t.y) * (1 << 23) + __float_as_int(r.y));
    return r;
}

// exp2_poly2 with exact zeros: anything below 2^-120 (a row whose lse is +inf, i.e. one that
// does not exist or saw no key) gives 0, as MUFU's 2^-inf does.
__device__ __forceinline__ float2 exp2_poly2_zero(float2 x) {
    float2 r = exp2_poly2(x);
    r.x = x.x < -120.f ? 0.f : r.x;
    r.y = x.y < -120.f ? 0.f : r.y;
    return r;
}

// Shared-memory matrix descriptor for a 128-byte swizzled tile (sm_100 format: version 1
// at bit 46, layout type 2 = SWIZZLE_128B at bit 61). Offsets in bytes.
__device__ __forceinline__ uint64_t smem_desc(uint32_t saddr, uint32_t lbo, uint32_t sbo) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((saddr & 0x3FFFFu) >> 4);
    d |= static_cast<uint64_t>(lbo >> 4) << 16;
    d |= static_cast<uint64_t>(sbo >> 4) << 32;
    d |= 1ull << 46;
    d |= 2ull << 61;
    return d;
}

// Instruction descriptor of kind::f16: fp32 accumulator, bf16 A and B, A K-major, B
// K-major or MN-major, M = 128.
__host__ __device__ constexpr uint32_t instr_desc(int n, bool b_mn_major) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((b_mn_major ? 1u : 0u) << 16) |
           (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(kBM >> 4) << 24);
}


// ---- host side (fwd_tc5.cu) -----------------------------------------------------------------

// Order of the row / head / batch dims by stride, as the tensor map wants them ascending.
struct DimOrder {
    int slot_of[3];  // slot (1..3) of row, head, batch
};

// Pinned, device-mapped status word: kernels record a bounded wait that ran out there.
int* status_word(int** device_view);
// Tensor map of a bf16 operand [rows, heads, batch] x d with the given element strides
// (row, head, batch), 128-byte swizzle, boxes of 64 columns x box_rows rows.
bool encode_map(
    CUtensorMap* map, const void* base, int d, int64_t rows, int64_t heads, int64_t batch,
    const int64_t strides[3], const DimOrder& order, int box_rows, const char** why);
// (batch, head, row) strides -> (row, head, batch) with size-1 dims given a valid stride.
bool operand_layout(
    const void* base, int64_t rows, int64_t heads, int64_t batch, const int64_t in[3],
    int64_t out[3], const char** why);
DimOrder order_of(const int64_t strides[3]);
// Optional profiling buffer (ktt_b200_set_trace).
long long* trace_buffer();

}  // namespace tc5
}  // namespace ktt
