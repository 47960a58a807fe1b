// Prefill / training forward for head dim 64 on the Blackwell tensor path, built for the
// case where the exponentials, not the tensor cores, bound a key block (at D 64 a 128 x 128
// block needs 16,384 exponentials but only ~650 tensor-pipe cycles).
//
// One CTA per SM runs two independent streams; a stream works on one 128-row query tile at a
// time with ten warps:
//
//   8 row warps        thread (r, g) owns query row r and the keys [64 g, 64 g + 64) of a
//                      block: maximum of its half row in a first pass over the scores in
//                      tensor memory, exchanged with the row's other thread through shared
//                      memory; exponentials, row sum and P (bf16) in a second pass; lazy
//                      rescale of O (only when the maximum moved by more than 2^8: the lazy
//                      rescale of ktt_flash/compute.cpp, flash.md "row reference")
//   1 MMA warp         S = Q K^T of block j + 1 as soon as the rows have read S of block j,
//                      O += P V with P read from tensor memory
//   1 producer warp    TMA loads of Q and of the K / V ring (three stages), and the draw of
//                      the stream's work from a counter in global memory
//
// Why sixteen row warps: measured on B200, inside this kernel one warp alone drives the
// MUFU pipe at about half its rate, and two take ~1,500 cycles for a block's exponentials
// where four take ~2,000: the pass is MUFU-bound only with four row warps per scheduler,
// which with tensor memory for two tiles (2 x 256 columns) means two threads per row. (Tried
// and measured, not kept: making the two streams take turns at the exponential pass through
// a lock per scheduler - slower, and locks on four schedulers can wait on one another in a
// cycle; starting stream 1 late - the streams' phases made no difference; one pass over the
// scores with the reference checked every 16 columns and P rescaled in tensor memory when it
// moves - without any check the block period falls by only 10 %, and the check costs more
// than that; ex2.approx.f16x2 for two exponentials per MUFU instruction - it issues at half
// rate, 16.8 cycles per instruction and scheduler against 8.2.)
// Tensor memory per stream (256 columns): S [0,128), P [128,192) as packed bf16 pairs,
// O [192,256).
//
// Work: a unit is a query tile of one (batch, head). Launches with many tiles per SM give
// each stream its own tiles. Launches with few (the 224 tiles of a 2,048-token, 14-head
// prefill on 148 SMs) run "dual": the two streams of a CTA share a tile, stream 0 taking the
// first half of its key blocks and stream 1 the second, so that the longest tile's serial
// chain is halved; stream 0's row warps then read stream 1's unnormalised O and (m, l)
// straight out of tensor memory and add the halves up (always half 0 then half 1: the
// result does not depend on timing). Tiles are drawn, longest first, from a counter in a
// small workspace; the last drawer resets it. Without a workspace the deal is fixed.
//
// Arithmetic contract as in the reference's flash forward (ktt_flash/compute.cpp:193-491):
// base-2 softmax with fp32 statistics, P rounded to bf16 before P V, fp32 accumulation,
// O / l and lse = ln2 (m + log2 l) at the end. The reference maximum a block is measured
// against is the row's maximum rounded up to bf16 precision (the two threads of a row
// exchange 16 bits each); any value at or above the maximum gives the same result up to
// rounding, and lse is computed from the value used.
//
// Every wait on an mbarrier is bounded: when one runs out the CTA records a code in a
// host-visible status word, stops waiting everywhere, frees its tensor memory and exits.
// Launched with programmatic stream serialization: everything before `griddepcontrol.wait`
// (barrier set-up, tensor-memory allocation, tensor-map prefetch) may overlap the tail of
// the previous kernel in the stream.
#include <cstdlib>
#include <mutex>
#include <type_traits>

#include "tc5.cuh"

namespace ktt {
using namespace tc5;
namespace {

constexpr float kRowRescaleGap = 8.f;  // log2 units

struct RowPlan {
    static constexpr int D = 64;
    static constexpr int kStreams = 2;
    static constexpr int kRowWarps = 8;                       // per stream: 2 column halves x 4 lane quarters
    static constexpr int kThreads = 32 * kStreams * (kRowWarps + 2);
    static constexpr int kTile = 128 * 128;   // one [128][64] bf16 tile, 128-byte rows, swizzled
    static constexpr int kStages = 3;
    // Tiles of a stream (1024-byte aligned): Q, K ring, V ring.
    static constexpr int kQ = 0;
    static constexpr int kK = kQ + kTile;
    static constexpr int kV = kK + kStages * kTile;
    static constexpr int kTileBytes = kV + kStages * kTile;   // per stream
    // Small areas of a stream, after both streams' tiles.
    static constexpr int kMaskRow = 0;            // float [128]: a block's mask terms
    static constexpr int kPairWords = 512;        // 512 bytes: what the two threads of a row exchange
    static constexpr int kBars = 1024;
    static constexpr int kBarBytes = 320;
    static constexpr int kSmallBytes = kBars + kBarBytes;
    static constexpr int kBytes = kStreams * (kTileBytes + kSmallBytes);
    static_assert(kBytes <= 232448, "shared memory per CTA");
    static constexpr int kTmemCols = 256;                // per stream
    static constexpr int kTmemP = 128;
    static constexpr int kTmemO = 192;
    // Exponentials per 8 pairs that take the FMA-pipe polynomial instead of MUFU.
#ifndef KTT_ROW_POLY_PAIRS
#define KTT_ROW_POLY_PAIRS 2
#endif
    static constexpr int kPolyPairs = KTT_ROW_POLY_PAIRS;
    // barrier indices
    static constexpr int bQFull = 0;
    static constexpr int bQFree = 1;
    static constexpr int bOFree = 2;
    static constexpr int bSFull = 3;
    static constexpr int bSFree = 4;
    static constexpr int bPFull = 5;
    static constexpr int bPVDone = 6;
    static constexpr int bKFull = 7;                    // + stage
    static constexpr int bVFull = bKFull + kStages;     // + stage
    static constexpr int bKVEmpty = bVFull + kStages;   // + stage
    static constexpr int bWorkFull = bKVEmpty + kStages;  // + slot
    static constexpr int bWorkFree = bWorkFull + 2;       // + slot
    static constexpr int bMaskFree = bWorkFree + 2;       // every row thread has read the mask row
    static constexpr int bMaskFull = bMaskFree + 1;       // the mask row is written
    static constexpr int bPair = bMaskFull + 1;           // + lane quarter: the two warps that share rows
    static constexpr int bDualReady = bPair + 4;          // stream 1's half of a shared tile is final in tensor memory
    static constexpr int bCount = bDualReady + 1;
    static_assert(bCount <= 32, "one barrier per lane at set-up");
    static_assert(bCount * 8 + 64 <= kBarBytes, "barrier area");
};

// Workspace (bytes): {int32 next tile, int32 drawers finished}, zero before the first use and
// left zero by every launch.
constexpr int64_t kRowHeaderBytes = 256;

struct RowParams {
    AttnParams a;
    int* status;
    int dim_of[3][3];
    long long* trace;
    int q_tiles;
    int units;          // tiles = heads * batch * q_tiles
    int dual;           // the two streams of a CTA share each tile (few tiles per SM)
    int* work_counter;  // null: a fixed deal
    int* done_counter;
    int grouped;        // tile order (decode_unit): 1 when K / V exceed what L2 keeps (needs the counter)
    Divisor by_heads, by_batch, by_kv_heads, by_group, by_per_pair;   // group: query heads per K/V head; per_pair: q_tiles * group
    // Optional (ktt_b200_set_dump, traced instantiation only): the tile (dump_b, dump_h, first row
    // dump_q0) writes what its row threads hold to `dump`: per key block kDumpBlock floats (the
    // exponents x = logit - reference [128][128], P = 2^x as the bf16 fed to P V [128][128], the
    // reference maximum of each half row [2][128]), then, behind dump_blocks blocks, the
    // unnormalised O [128][64], the final maximum [128] and the row sum [128].
    float* dump;
    int dump_b, dump_h, dump_q0, dump_blocks;
};
constexpr int kDumpBlock = 2 * 128 * 128 + 2 * 128;
constexpr int kDumpTail = 128 * 64 + 2 * 128;

struct Unit {
    int b, h, q0;
    int j0, j1;      // key blocks [j0, j1) this stream works on
    int nblocks;     // key blocks of the whole tile
    SeqInfo si;
    bool valid;
};

// Tiles are ordered heads fastest, longest causal tiles first (consecutive tiles are the
// heads of one GQA group on the same keys). In dual mode stream 0 takes the first half of a
// tile's key blocks (the larger one when the count is odd) and stream 1 the rest.
__device__ __forceinline__ Unit decode_unit(const RowParams& tp, int u, int stream) {
    const AttnParams& p = tp.a;
    Unit k;
    int qb;
    if (tp.grouped) {
        // All query tiles of one (batch, K / V head) follow one another, longest first, the
        // heads of the GQA group fastest: the tiles in flight share a few pairs' K / V in L2.
        const int group = static_cast<int>(tp.by_group.d);
        const int pair = div_by(u, tp.by_per_pair), r = u - pair * static_cast<int>(tp.by_per_pair.d);
        const int tile = div_by(r, tp.by_group);
        k.b = div_by(pair, tp.by_kv_heads);
        k.h = (pair - k.b * p.kv_heads) * group + (r - tile * group);
        qb = tp.q_tiles - 1 - tile;
    } else {
        const int t = div_by(u, tp.by_heads), level = div_by(t, tp.by_batch);
        k.h = u - t * p.heads;
        k.b = t - level * p.batch;
        qb = tp.q_tiles - 1 - level;
    }
    k.si = seq_info(p, k.b);
    k.q0 = qb * kBM;
    k.valid = k.q0 < k.si.lq;
    int kend = k.si.klen;
    if (p.causal) kend = min(kend, min(k.q0 + kBM, k.si.lq) - 1 + k.si.shift + 1);
    k.nblocks = (k.valid && kend > 0) ? (kend + kBN - 1) / kBN : 0;
    k.j0 = 0;
    k.j1 = k.nblocks;
    if (tp.dual) {
        const int half = (k.nblocks + 1) >> 1;
        if (stream == 0) {
            k.j1 = half;
        } else {
            k.j0 = half;
        }
    }
    return k;
}

__device__ __forceinline__ int snake(int round, int cta, int ctas) {
    return round * ctas + ((round & 1) ? ctas - 1 - cta : cta);
}

template <bool kTrace>
__device__ __forceinline__ void rzone(const RowParams& tp, bool who, int j, int slot) {
    if constexpr (kTrace) {
        if (who && j < 64) tp.trace[j * 8 + slot] = clock64();
    }
}

__device__ __forceinline__ float max3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));   // one three-input instruction
    return d;
}
// A float rounded towards +inf to bf16 precision, as its upper 16 bits.
__device__ __forceinline__ uint32_t round_up_bf16(float x) {
    const uint32_t bits = __float_as_uint(x);
    return (x >= 0.f ? bits + 0xFFFFu : bits) >> 16;
}

template <bool kTrace, bool kMask>
__global__ void __launch_bounds__(RowPlan::kThreads, 1) fwd_row_kernel(
    const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
    const __grid_constant__ CUtensorMap map_v, const RowParams tp) {
    using P = RowPlan;
    constexpr int D = P::D;
    constexpr int S = P::kStreams;
    constexpr int RW = P::kRowWarps;
    extern __shared__ __align__(1024) unsigned char smem_all[];
    if (smem_u32(smem_all) & 1023u) {   // swizzled tiles need a 1024-byte aligned base
        if (threadIdx.x == 0) atomicCAS_system(tp.status, 0, 901);
        return;
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // Role and stream of this warp: row warps [0, 8 S), MMA warps [8 S, 9 S), producers [9 S, 10 S).
    const bool is_row = warp < RW * S, is_mma = !is_row && warp < (RW + 1) * S;
    const bool is_producer = !is_row && !is_mma;
    const int stream = is_row ? warp / RW : (is_mma ? warp - RW * S : warp - (RW + 1) * S);
    const int quarter = warp & 3;        // row warps: TMEM lane quarter (and scheduler)
    const int group = (warp >> 2) & 1;   // row warps: which half of a block's keys
    unsigned char* tiles = smem_all + stream * P::kTileBytes;
    unsigned char* small = smem_all + S * P::kTileBytes + stream * P::kSmallBytes;
    const uint32_t sbase = smem_u32(tiles);
    long long cta_t0 = 0;
    if (kTrace && is_mma && lane == 0) asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(cta_t0));
    const uint32_t bars = smem_u32(small) + P::kBars;
    auto bar = [&](int i) { return bars + 8u * i; };
    // CTA-wide words live in stream 0's small area: the abort flag and the tensor-memory base.
    unsigned char* shared0 = smem_all + S * P::kTileBytes + P::kBars + P::bCount * 8;
    volatile int* abort_flag = reinterpret_cast<volatile int*>(shared0);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(shared0 + 8);
    volatile int* work_slot = reinterpret_cast<volatile int*>(small + P::kBars + P::bCount * 8 + 16);  // [2], per stream (bytes 16..23)

    const AttnParams& p = tp.a;

    if (is_producer) {
        if (lane < P::bCount) {
            uint32_t count = 1;
            if (lane == P::bDualReady) count = RW;
            if (lane == P::bOFree || lane == P::bSFree || lane == P::bPFull || lane == P::bMaskFree ||
                lane == P::bMaskFull) count = RW;                                 // one arrival per row warp
            if (lane >= P::bWorkFree && lane < P::bWorkFree + 2) {
                count = RW + 1;                                     // row warps and the MMA warp ...
                if (tp.dual && stream == 1) count = RW + 2;         // ... and, in dual mode, stream 1's producer
            }
            if (lane >= P::bPair && lane < P::bPair + 4) count = 2;
            mbar_init(bar(lane), count);
        }
        if (lane == 0 && stream == 0) {
            asm volatile("prefetch.tensormap [%0];" ::"l"(&map_q) : "memory");
            asm volatile("prefetch.tensormap [%0];" ::"l"(&map_k) : "memory");
            asm volatile("prefetch.tensormap [%0];" ::"l"(&map_v) : "memory");
            *abort_flag = 0;
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        fence_async_smem();
        __syncwarp();
    } else if (is_mma && stream == 0) {
        tmem_alloc(smem_u32(tmem_slot), P::kTmemCols * S);
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    // The next kernel in the stream may start its own set-up now; nothing of this launch has
    // touched global memory yet, and nothing will before the previous kernel has completed.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");

    const uint32_t tmem_base = *tmem_slot;
    const uint32_t tmem = tmem_base + stream * P::kTmemCols;
    const uint32_t tmem_p = tmem + P::kTmemP;
    const uint32_t tmem_o = tmem + P::kTmemO;

    auto coords = [&](int operand, int row, int head, int batch, int (&c)[4]) {
        c[tp.dim_of[operand][0]] = row;
        c[tp.dim_of[operand][1]] = head;
        c[tp.dim_of[operand][2]] = batch;
    };

    int blocks_done = 0;

    // Barriers and work slots of the other stream (dual mode: stream 0's producer feeds both
    // queues, stream 0's rows read stream 1's half).
    unsigned char* small_other = smem_all + S * P::kTileBytes + (stream ^ 1) * P::kSmallBytes;
    const uint32_t bars_other = smem_u32(small_other) + P::kBars;
    auto bar_other = [&](int i) { return bars_other + 8u * i; };
    volatile int* work_slot_other = reinterpret_cast<volatile int*>(small_other + P::kBars + P::bCount * 8 + 16);

    // The n-th unit of this stream: -1 = no more, -2 = nothing at this position.
    const bool dynamic = tp.work_counter != nullptr;
    const bool dual = tp.dual != 0;
    const int lanes_total = dual ? gridDim.x : gridDim.x * S;                 // dealing positions
    const int my_lane = dual ? blockIdx.x : blockIdx.x * S + stream;
    auto static_unit = [&](int n) -> int {
        if (static_cast<int64_t>(n) * lanes_total >= tp.units) return -1;
        const int u = snake(n, my_lane, lanes_total);
        return u < tp.units ? u : -2;
    };
    auto take_unit = [&](int n, bool& ok) -> int {   // every role but the drawing producer
        if (!dynamic) return static_unit(n);
        const int slot = n & 1;
        ok = __all_sync(0xffffffffu, mbar_wait(bar(P::bWorkFull + slot), (n >> 1) & 1, abort_flag, 130 + slot, tp.status));
        if (!ok) return -1;
        const int u = work_slot[slot];
        mbar_arrive_warp(bar(P::bWorkFree + slot));
        return u;
    };
    auto draw_unit = [&](int n, bool& ok) -> int {   // producer warp, converged
        if (!dynamic) return static_unit(n);
        if (dual && stream == 1) return take_unit(n, ok);   // stream 0's producer draws for both
        const int slot = n & 1;
        if (n >= 2) {
            ok = __all_sync(0xffffffffu, mbar_wait(bar(P::bWorkFree + slot), ((n >> 1) - 1) & 1, abort_flag, 120 + slot, tp.status));
            if (ok && dual) ok = __all_sync(0xffffffffu, mbar_wait(bar_other(P::bWorkFree + slot), ((n >> 1) - 1) & 1, abort_flag, 122 + slot, tp.status));
            if (!ok) return -1;
        }
        int u;
        while (true) {
            int pos = 0;
            if (lane == 0) pos = atomicAdd(tp.work_counter, 1);
            pos = __shfl_sync(0xffffffffu, pos, 0);
            if (pos >= tp.units) {
                u = -1;
                break;
            }
            u = pos;
            if (!dual && !tp.grouped) {
                // Tiles are sorted by decreasing work. The first draws (one per stream, all at
                // once when the kernel starts) alternate between the front and the back of the
                // list, so the two streams of an SM start with a long tile and a short one; the
                // draws after that walk the middle in decreasing order.
                const int wave = min(lanes_total, tp.units) & ~1;
                u = pos < wave ? ((pos & 1) ? tp.units - 1 - (pos >> 1) : (pos >> 1)) : pos - (wave >> 1);
            }
            if (decode_unit(tp, u, stream).valid) break;
        }
        if (lane == 0) {
            work_slot[slot] = u;
            if (dual) work_slot_other[slot] = u;
            __threadfence_block();
            mbar_arrive(bar(P::bWorkFull + slot));
            if (dual) mbar_arrive(bar_other(P::bWorkFull + slot));
        }
        return u;
    };

    if (is_producer) {
        // ---------------- producer (whole warp, converged) ----------------
        int uidx = 0, blk = 0;
        bool ok = true;
        // In the grouped order units are fetched one ahead, so that the trip to the counter
        // (and the positions past the end of short sequences a draw skips) hides behind a
        // whole unit's loads. Otherwise a unit is drawn when its loads start: committing a
        // unit earlier evens the streams out less well at the end (measured: 613 against 571
        // TFLOP/s on B 2, S 4096).
        const bool ahead = tp.grouped != 0;
        int u_next = ahead ? draw_unit(0, ok) : 0;
        for (int n = 0; ok; ++n) {
            const int u = ahead ? u_next : draw_unit(n, ok);
            if (u == -1) break;
            if (ahead) u_next = draw_unit(n + 1, ok);
            if (!ok) break;
            if (u == -2) continue;
            const Unit k = decode_unit(tp, u, stream);
            const int nb = k.j1 - k.j0;
            if (!k.valid || nb <= 0) continue;
            const int hk = div_by(k.h, tp.by_group);
            int c[4], cv[4];
            const int batch = p.cu_q ? 0 : k.b;
            c[0] = cv[0] = 0;
            if (uidx > 0) {
                ok = __all_sync(0xffffffffu, mbar_wait(bar(P::bQFree), (uidx - 1) & 1, abort_flag, 110, tp.status));
                if (!ok) break;
            }
            coords(0, k.si.q_off + k.q0, k.h, batch, c);
            mbar_expect_tx(bar(P::bQFull), P::kTile);
            tma_load_4d(sbase + P::kQ, &map_q, bar(P::bQFull), 0, c[1], c[2], c[3]);
            for (int jj = 0; jj < nb; ++jj) {
                const int gb = blk + jj, st = gb % P::kStages;
                if (gb >= P::kStages) {
                    ok = __all_sync(0xffffffffu, mbar_wait(bar(P::bKVEmpty + st), ((gb / P::kStages) - 1) & 1, abort_flag, 100 + st, tp.status));
                    if (!ok) break;
                }
                coords(1, k.si.k_off + (k.j0 + jj) * kBN, hk, batch, c);
                coords(2, k.si.k_off + (k.j0 + jj) * kBN, hk, batch, cv);
                mbar_expect_tx(bar(P::bKFull + st), P::kTile);
                tma_load_4d(sbase + P::kK + st * P::kTile, &map_k, bar(P::bKFull + st), 0, c[1], c[2], c[3]);
                mbar_expect_tx(bar(P::bVFull + st), P::kTile);
                tma_load_4d(sbase + P::kV + st * P::kTile, &map_v, bar(P::bVFull + st), 0, cv[1], cv[2], cv[3]);
            }
            blk += nb;
            ++uidx;
        }
        if (*abort_flag) {
            const long long t0 = clock64();
            while (clock64() - t0 < 4000000) {   // let copies in flight land
            }
        } else if (dynamic && lane == 0 && !(dual && stream == 1)) {
            // This producer draws no more. The last stream to say so puts the counters back to
            // zero for the next launch.
            __threadfence();
            const int done = atomicAdd(tp.done_counter, 1);
            if (done == lanes_total - 1) {   // lanes_total = the number of drawing producers
                *tp.work_counter = 0;
                *tp.done_counter = 0;
                __threadfence();
            }
        }
    } else if (is_mma) {
        // ---------------- MMA issuer (whole warp, converged) ----------------
        constexpr uint32_t idesc_s = instr_desc(kBN, false);
        constexpr uint32_t idesc_o = instr_desc(D, true);
        const uint64_t q_desc = smem_desc(sbase + P::kQ, 16, 1024);
        const uint64_t k_desc = smem_desc(sbase + P::kK, 16, 1024);
        const uint64_t v_desc = smem_desc(sbase + P::kV, P::kTile, 1024);
        int uidx = 0, blk = 0;
        bool ok = true;
        // S = Q K^T of global block gb; `last` = the unit's last one, after which Q is free.
        auto issue_s = [&](int gb, bool last) {
            const uint64_t kd = k_desc + static_cast<uint64_t>(((gb % P::kStages) * P::kTile) >> 4);
#pragma unroll
            for (int ks = 0; ks < D / 16; ++ks) {
                tc_mma(tmem, q_desc + ((ks * 32) >> 4), kd + ((ks * 32) >> 4), idesc_s, ks > 0);
            }
            tc_commit(bar(P::bSFull));
            if (last) tc_commit(bar(P::bQFree));
        };
        for (int n = 0; ok; ++n) {
            const int u = take_unit(n, ok);
            if (u == -1) break;
            if (u == -2) continue;
            const Unit k = decode_unit(tp, u, stream);
            const int nb = k.j1 - k.j0;
            if (!k.valid || nb <= 0) continue;
            ok = __all_sync(0xffffffffu, mbar_wait(bar(P::bQFull), uidx & 1, abort_flag, 200, tp.status));
            if (!ok) break;
            {
                // First S of the unit: the rows have long read the previous unit's last S.
                const int gb = blk;
                ok = __all_sync(0xffffffffu, mbar_wait(bar(P::bKFull + gb % P::kStages), (gb / P::kStages) & 1, abort_flag, 210, tp.status));
                if (ok && gb > 0) ok = __all_sync(0xffffffffu, mbar_wait(bar(P::bSFree), (gb - 1) & 1, abort_flag, 211, tp.status));
                if (!ok) break;
                tc_fence_after();
                issue_s(gb, nb == 1);
            }
            for (int jj = 0; ok && jj < nb; ++jj) {
                const int gb = blk + jj, st = gb % P::kStages;
                if (jj + 1 < nb) {
                    // S of the next block goes out as soon as the rows hold this block's scores
                    // in registers, ahead of this block's P V.
                    const int g2 = gb + 1;
                    ok = __all_sync(0xffffffffu, mbar_wait(bar(P::bKFull + g2 % P::kStages), (g2 / P::kStages) & 1, abort_flag, 220, tp.status));
                    if (ok) ok = __all_sync(0xffffffffu, mbar_wait(bar(P::bSFree), gb & 1, abort_flag, 221, tp.status));
                    if (!ok) break;
                    tc_fence_after();
                    issue_s(g2, jj + 2 == nb);
                }
                if (jj == 0 && uidx > 0) {
                    // O is free once the previous unit's epilogue has read it.
                    ok = __all_sync(0xffffffffu, mbar_wait(bar(P::bOFree), (uidx - 1) & 1, abort_flag, 250, tp.status));
                    if (!ok) break;
                }
                ok = __all_sync(0xffffffffu, mbar_wait(bar(P::bVFull + st), (gb / P::kStages) & 1, abort_flag, 230, tp.status));
                if (!ok) break;
                if (p.key_lengths) {
                    // Cache rows past the length may hold anything and 0 x inf would poison the
                    // output: blank those value rows in the tile (TMA only blanks rows past the
                    // end of the tensor).
                    const int valid = k.si.klen - (k.j0 + jj) * kBN;
                    if (valid < kBN) {
                        const int rows = kBN - (valid > 0 ? valid : 0), first = kBN - rows;
                        unsigned char* vt = tiles + P::kV + st * P::kTile;
                        for (int idx = lane; idx < rows * 8; idx += 32) {
                            *reinterpret_cast<uint4*>(vt + (first + idx / 8) * 128 + (idx % 8) * 16) = make_uint4(0u, 0u, 0u, 0u);
                        }
                        fence_async_smem();
                        __syncwarp();
                    }
                }
                ok = __all_sync(0xffffffffu, mbar_wait(bar(P::bPFull), gb & 1, abort_flag, 240, tp.status));
                if (!ok) break;
                tc_fence_after();
                const uint64_t vd = v_desc + static_cast<uint64_t>((st * P::kTile) >> 4);
#pragma unroll
                for (int ks = 0; ks < kBN / 16; ++ks) {
                    // A: P, 8 TMEM columns per 16 keys. B: V MN-major, 16 keys = 16 rows of 128 B.
                    tc_mma_ts(tmem_o, tmem_p + ks * 8, vd + ((ks * 2048) >> 4), idesc_o, (jj > 0 || ks > 0) ? 1u : 0u);
                }
                tc_commit(bar(P::bPVDone));
                tc_commit(bar(P::bKVEmpty + st));
            }
            blk += nb;
            ++uidx;
        }
        blocks_done = blk;
    } else {
        // ---------------- rows: thread = (query row, half of a block's keys) ----------------
        const int row = quarter * 32 + lane;
        const uint32_t lane_addr = static_cast<uint32_t>(quarter * 32) << 16;
        const uint32_t s_addr = tmem + lane_addr + group * 64;
        const uint32_t p_addr = tmem_p + lane_addr + group * 32;
        const uint32_t o_addr = tmem_o + lane_addr + group * 32;   // this thread's 32 output columns
        int uidx = 0, blk = 0;
        uint32_t pair_uses = 0;   // phases of this quarter's pair barrier so far
        int didx = 0;             // tiles shared with the other stream so far (dual mode)
        bool ok = true;
        bool first_unit = true;
        const float* mrow = reinterpret_cast<const float*>(small + P::kMaskRow);
        unsigned char* pair_words = small + P::kPairWords;
        // The two warps that share rows meet (bounded, like every wait here).
        auto pair_meet = [&](int code) -> bool {
            mbar_arrive_warp(bar(P::bPair + quarter));
            const bool met = __all_sync(0xffffffffu, mbar_wait(bar(P::bPair + quarter), pair_uses & 1, abort_flag, code, tp.status));
            ++pair_uses;
            return met;
        };

        for (int n = 0; ok; ++n) {
            const int u = take_unit(n, ok);
            if (u == -1) break;
            if (u == -2) continue;
            // What the block loop needs of the unit, as a few scalars: the unit is decoded again
            // for the epilogue rather than kept in registers across the loop.
            int nb, col0, row_limit;
            bool dumping = false;   // traced instantiation: this is the tile whose values are written out
            int dump_j0 = 0;
            int mask_b = 0, mask_h = 0, mask_koff = 0, mask_klen = 1;
            {
                const Unit k = decode_unit(tp, u, stream);
                if (!k.valid) continue;
                const int qi = k.q0 + row;
                if (k.j1 <= k.j0 && k.nblocks > 0) continue;   // dual mode, one-block tile: stream 1 has nothing to do
                if (k.nblocks == 0) {
                    // No key is visible to this tile: zeros, lse = -inf. No barrier is involved.
                    if (qi < k.si.lq && (!dual || stream == 0)) {
                        __nv_bfloat16* og = p.out + k.b * p.os[0] + k.h * p.os[1] + static_cast<int64_t>(k.si.q_off + qi) * p.os[2] + group * 32;
#pragma unroll
                        for (int c = 0; c < 4; ++c) *reinterpret_cast<uint4*>(og + c * 8) = make_uint4(0u, 0u, 0u, 0u);
                        if (group == 0 && p.lse) p.lse[k.b * p.ls[0] + k.h * p.ls[1] + (k.si.q_off + qi) * p.ls[2]] = -INFINITY;
                    }
                    continue;
                }
                nb = k.j1 - k.j0;
                if constexpr (kTrace) {
                    dumping = tp.dump && k.b == tp.dump_b && k.h == tp.dump_h && k.q0 == tp.dump_q0;
                    dump_j0 = k.j0;
                }
                col0 = k.j0 * kBN + group * 64;   // first key column of this thread in the unit's first block
                row_limit = k.si.klen;
                if (p.causal) row_limit = min(row_limit, qi + k.si.shift + 1);
                if constexpr (kMask) {
                    mask_b = k.b;
                    mask_h = k.h;
                    mask_koff = k.si.k_off;
                    mask_klen = k.si.klen;
                }
            }
            const bool tracer = kTrace && tp.trace && first_unit && row == 0 && group == 0 && blockIdx.x == 0 && stream == 0;
            float m_ref = -INFINITY;
            float2 l2[2] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
            const float sc1 = kMask ? 1.f : p.scale_log2;   // masked logits are scaled when read

            for (int jj = 0; ok && jj < nb; ++jj) {
                const int gb = blk + jj;
                const int limit = row_limit - col0 - jj * kBN;   // my columns [0, limit) are visible
                const bool whole = __all_sync(0xffffffffu, limit >= 64);
                if constexpr (kMask) {
                    // One thread per column fetches the block's mask terms; the rows share them
                    // through shared memory (bounded mbarriers, not bar.sync: a warp that gave
                    // up elsewhere must not strand the others here).
                    mbar_arrive_warp(bar(P::bMaskFree));
                    ok = __all_sync(0xffffffffu, mbar_wait(bar(P::bMaskFree), gb & 1, abort_flag, 340, tp.status));
                    if (!ok) break;
                    if (group == 0) {
                        const int col = max(min(col0 + jj * kBN + row, mask_klen - 1), 0);   // group 0: col0 is the block's first key
                        reinterpret_cast<float*>(small + P::kMaskRow)[row] =
                            mask_value(p, mask_b, mask_h, 0, static_cast<int64_t>(mask_koff) + col) * kLog2e;
                    }
                    mbar_arrive_warp(bar(P::bMaskFull));
                    ok = __all_sync(0xffffffffu, mbar_wait(bar(P::bMaskFull), gb & 1, abort_flag, 350, tp.status));
                    if (!ok) break;
                }
                ok = __all_sync(0xffffffffu, mbar_wait(bar(P::bSFull), gb & 1, abort_flag, 300, tp.status));
                if (!ok) break;
                tc_fence_after();
                rzone<kTrace>(tp, tracer, jj, 0);

                float sa[16], sb[16];
                auto logits = [&](float (&s)[16], int c) {   // in place: scale + mask term, visibility
                    if constexpr (kMask) {
#pragma unroll
                        for (int e4 = 0; e4 < 4; ++e4) {
                            const float4 t = reinterpret_cast<const float4*>(mrow)[group * 16 + c * 4 + e4];
                            s[e4 * 4] = fmaf(s[e4 * 4], p.scale_log2, t.x);
                            s[e4 * 4 + 1] = fmaf(s[e4 * 4 + 1], p.scale_log2, t.y);
                            s[e4 * 4 + 2] = fmaf(s[e4 * 4 + 2], p.scale_log2, t.z);
                            s[e4 * 4 + 3] = fmaf(s[e4 * 4 + 3], p.scale_log2, t.w);
                        }
                    }
                    if (!whole) {
#pragma unroll
                        for (int e = 0; e < 16; ++e) s[e] = (c * 16 + e) < limit ? s[e] : -INFINITY;
                    }
                };

                // ---- pass 1: the maximum of this thread's 64 logits ----
                float mx4[2] = {-INFINITY, -INFINITY};
                auto reduce32 = [&](float (&s)[32], int half) {
                    if constexpr (kMask) {
#pragma unroll
                        for (int e4 = 0; e4 < 8; ++e4) {
                            const float4 t = reinterpret_cast<const float4*>(mrow)[group * 16 + half * 8 + e4];
                            s[e4 * 4] = fmaf(s[e4 * 4], p.scale_log2, t.x);
                            s[e4 * 4 + 1] = fmaf(s[e4 * 4 + 1], p.scale_log2, t.y);
                            s[e4 * 4 + 2] = fmaf(s[e4 * 4 + 2], p.scale_log2, t.z);
                            s[e4 * 4 + 3] = fmaf(s[e4 * 4 + 3], p.scale_log2, t.w);
                        }
                    }
                    if (!whole) {
#pragma unroll
                        for (int e = 0; e < 32; ++e) s[e] = (half * 32 + e) < limit ? s[e] : -INFINITY;
                    }
#pragma unroll
                    for (int e = 0; e < 32; e += 4) {
                        mx4[0] = max3(mx4[0], s[e], s[e + 1]);
                        mx4[1] = max3(mx4[1], s[e + 2], s[e + 3]);
                    }
                };
                {
                    float w[32];
                    tmem_ld32(s_addr, w);
                    tmem_wait_ld();
                    reduce32(w, 0);
                    tmem_ld32(s_addr + 32, w);
                    tmem_wait_ld();
                    reduce32(w, 1);
                }
                // The row's two threads exchange their maxima (16 bits each, rounded up).
                const uint32_t mine16 = round_up_bf16(fmaxf(mx4[0], mx4[1]) * sc1);
                reinterpret_cast<volatile uint16_t*>(pair_words)[group * 128 + row] = static_cast<uint16_t>(mine16);
                ok = pair_meet(360);
                if (!ok) break;
                const uint32_t other16 = reinterpret_cast<volatile uint16_t*>(pair_words)[(group ^ 1) * 128 + row];
                const float mx = fmaxf(__uint_as_float(mine16 << 16), __uint_as_float(other16 << 16));
                rzone<kTrace>(tp, tracer, jj, 1);

                // Lazy rescale: move the reference only when this block exceeds it by 2^8. Both
                // threads of a row take the same decision from the same numbers; each rescales
                // its own 32 columns of O.
                const bool move = mx > m_ref + kRowRescaleGap;
                if (__any_sync(0xffffffffu, move)) {
                    float f = 1.f;
                    if (move) {
                        f = fast_exp2(m_ref - mx);   // 0 on the first block
                        m_ref = mx;
                        l2[0] = __fmul2_rn(l2[0], make_float2(f, f));
                        l2[1] = __fmul2_rn(l2[1], make_float2(f, f));
                    }
                    if (jj > 0) {
                        // O holds blocks [0, jj): wait for the previous block's P V.
                        ok = __all_sync(0xffffffffu, mbar_wait(bar(P::bPVDone), (gb - 1) & 1, abort_flag, 310, tp.status));
                        if (!ok) break;
                        tc_fence_after();
#pragma unroll 1
                        for (int c = 0; c < 2; ++c) {
                            float o[16];
                            tmem_ld16(o_addr + c * 16, o);
                            tmem_wait_ld();
#pragma unroll
                            for (int e = 0; e < 16; ++e) o[e] *= f;
                            tmem_st16(o_addr + c * 16, reinterpret_cast<const uint32_t*>(o));
                        }
                        tmem_wait_st();
                    }
                }
                const float m_use = (m_ref == -INFINITY) ? 0.f : m_ref;
                const float2 sc2 = make_float2(sc1, sc1), nm2 = make_float2(-m_use, -m_use);

                // ---- pass 2: P = 2^(logit - m) as packed bf16, 16 columns at a time ----
                // (Traced instantiation, the dumped tile only: the exponents and P as they are,
                // and the reference maximum this block is measured against.)
                float* dump_block = nullptr;
                if constexpr (kTrace) {
                    if (dumping && dump_j0 + jj < tp.dump_blocks) {
                        dump_block = tp.dump + static_cast<int64_t>(dump_j0 + jj) * kDumpBlock;
                        dump_block[2 * 128 * 128 + group * 128 + row] = m_ref;
                    }
                }
                auto dump_pair = [&](int c, int e, const float2& x, uint32_t packed) {
                    if constexpr (kTrace) {
                        if (dump_block) {
                            float* at = dump_block + row * 128 + group * 64 + c * 16 + 2 * e;
                            at[0] = x.x;
                            at[1] = x.y;
                            at[128 * 128] = __uint_as_float(packed << 16);
                            at[128 * 128 + 1] = __uint_as_float(packed & 0xffff0000u);
                        }
                    }
                };
                auto exps = [&](float (&s)[16], int c, uint32_t (&wv)[8]) {
                    logits(s, c);
                    if (whole) {
#pragma unroll
                        for (int e = 0; e < 8; ++e) {
                            const float2 x = __ffma2_rn(make_float2(s[2 * e], s[2 * e + 1]), sc2, nm2);
                            float2 pr;
                            // The polynomial pairs sit at the start of odd chunks and at the end
                            // of even ones, so MUFU and FMA work alternate along the row.
                            if ((c & 1) ? (e < P::kPolyPairs) : (e >= 8 - P::kPolyPairs)) {
                                pr = exp2_poly2(x);
                            } else {
                                pr.x = fast_exp2(x.x);
                                pr.y = fast_exp2(x.y);
                            }
                            l2[e & 1] = __fadd2_rn(l2[e & 1], pr);
                            wv[e] = pack_bf16(pr.x, pr.y);
                            dump_pair(c, e, x, wv[e]);
                        }
                    } else {
                        // Hidden columns take MUFU, whose 2^-inf is exactly 0.
#pragma unroll
                        for (int e = 0; e < 8; ++e) {
                            const float2 x = __ffma2_rn(make_float2(s[2 * e], s[2 * e + 1]), sc2, nm2);
                            const float2 pr = make_float2(fast_exp2(x.x), fast_exp2(x.y));
                            l2[e & 1] = __fadd2_rn(l2[e & 1], pr);
                            wv[e] = pack_bf16(pr.x, pr.y);
                            dump_pair(c, e, x, wv[e]);
                        }
                    }
                };
                uint32_t wv[8];
                tmem_ld16(s_addr, sa);
                tmem_wait_ld();
                rzone<kTrace>(tp, tracer, jj, 4);
                tmem_ld16(s_addr + 16, sb);
                exps(sa, 0, wv);
                rzone<kTrace>(tp, tracer, jj, 5);
                if (jj > 0) {
                    // The P columns are free once the previous block's P V has read them.
                    ok = __all_sync(0xffffffffu, mbar_wait(bar(P::bPVDone), (gb - 1) & 1, abort_flag, 320, tp.status));
                    if (!ok) break;
                    tc_fence_after();
                } else if (dual && stream == 1 && uidx > 0) {
                    // ... and, on a tile's first block, once stream 0's rows have read the (m, l)
                    // this stream left there for the previous shared tile.
                    ok = __all_sync(0xffffffffu, mbar_wait(bar(P::bOFree), (uidx - 1) & 1, abort_flag, 321, tp.status));
                    if (!ok) break;
                    tc_fence_after();
                }
                rzone<kTrace>(tp, tracer, jj, 6);
                tmem_st8(p_addr, wv);
                tmem_wait_ld();
                rzone<kTrace>(tp, tracer, jj, 7);
                tmem_ld16(s_addr + 32, sa);
                exps(sb, 1, wv);
                tmem_st8(p_addr + 8, wv);
                tmem_wait_ld();
                tmem_ld16(s_addr + 48, sb);
                exps(sa, 2, wv);
                tmem_st8(p_addr + 16, wv);
                tmem_wait_ld();
                // All of this thread's scores are in registers: the next S may overwrite them.
                tc_fence_before();
                mbar_arrive_warp(bar(P::bSFree));
                exps(sb, 3, wv);
                rzone<kTrace>(tp, tracer, jj, 2);
                tmem_st8(p_addr + 24, wv);
                tmem_wait_st();
                tc_fence_before();
                mbar_arrive_warp(bar(P::bPFull));
                rzone<kTrace>(tp, tracer, jj, 3);
            }
            if (!ok) break;

            // ---- the unit's epilogue ----
            const Unit k = decode_unit(tp, u, stream);
            const SeqInfo& si = k.si;
            const int qi = k.q0 + row;
            const bool real = qi < si.lq;
            __nv_bfloat16* og = p.out + k.b * p.os[0] + k.h * p.os[1] + static_cast<int64_t>(si.q_off + qi) * p.os[2] + group * 32;
            const int last = blk + nb - 1;
            ok = __all_sync(0xffffffffu, mbar_wait(bar(P::bPVDone), last & 1, abort_flag, 330, tp.status));
            if (!ok) break;
            tc_fence_after();
            rzone<kTrace>(tp, tracer, 60, 0);
            float o[32];
            tmem_ld32(o_addr, o);
            // The row sum: half 1 hands its part to half 0, which adds (always in this order)
            // and hands the total back.
            float l_row = (l2[0].x + l2[0].y) + (l2[1].x + l2[1].y);
            // The word of this row lies inside the 128 bytes that hold the maxima of this pair
            // of warps (16-bit words [half][row], 64 bytes per half and pair): the pair's own
            // meetings order every access to them. (Indexed by row as floats, the sums of one
            // pair lay over the maxima of another, which may already be in its next tile:
            // sixteen rows of a tile came out wrong once in a few hundred tiles.)
            volatile float* lsum = reinterpret_cast<volatile float*>(pair_words + (lane < 16 ? 0 : 256) + quarter * 64 + (lane & 15) * 4);
            if (group == 1) *lsum = l_row;
            ok = pair_meet(370);
            if (!ok) break;
            if (group == 0) {
                l_row += *lsum;
                *lsum = l_row;
            }
            ok = pair_meet(371);
            if (!ok) break;
            if (group == 1) l_row = *lsum;
            // Half 0 writes these words again in the next unit's first exchange: not before
            // half 1 has read the total.
            ok = pair_meet(372);
            if (!ok) break;
            tmem_wait_ld();
            tc_fence_before();
            // The next unit's P V may overwrite O; for stream 1's half of a shared tile that is
            // for stream 0's rows to say, after they have read it.
            if (!(dual && stream == 1 && k.nblocks > 1)) mbar_arrive_warp(bar(P::bOFree));
            rzone<kTrace>(tp, tracer, 60, 2);
            float m_row = m_ref;
            bool finish = true;
            if (dual && k.nblocks > 1) {
                // This tile's key blocks are shared by the CTA's two streams.
                if (stream == 1) {
                    // Leave (m, l) beside O in tensor memory (the P columns are idle now) and tell
                    // stream 0's rows; they free this stream's O when they have read it.
                    finish = false;
                    if (group == 0) {
                        const uint32_t ml[2] = {__float_as_uint(m_row), __float_as_uint(l_row)};
                        asm volatile("tcgen05.st.sync.aligned.32x32b.x2.b32 [%0], {%1, %2};"
                                     ::"r"(tmem_p + lane_addr), "r"(ml[0]), "r"(ml[1]) : "memory");
                        tmem_wait_st();
                    }
                    tc_fence_before();
                    mbar_arrive_warp(bar(P::bDualReady));
                } else {
                    ok = __all_sync(0xffffffffu, mbar_wait(bar_other(P::bDualReady), didx & 1, abort_flag, 380, tp.status));
                    if (!ok) break;
                    tc_fence_after();
                    rzone<kTrace>(tp, tracer, 60, 3);   // the other stream's half is in
                    const uint32_t other = tmem_base + P::kTmemCols;   // stream 1's columns
                    float o1[32];
                    uint32_t ml0, ml1;
                    tmem_ld32(other + P::kTmemO + lane_addr + group * 32, o1);
                    asm volatile("tcgen05.ld.sync.aligned.32x32b.x2.b32 {%0, %1}, [%2];"
                                 : "=r"(ml0), "=r"(ml1) : "r"(other + P::kTmemP + lane_addr) : "memory");
                    tmem_wait_ld();
                    rzone<kTrace>(tp, tracer, 60, 4);   // ... and in this thread's registers
                    tc_fence_before();
                    mbar_arrive_warp(bar_other(P::bOFree));   // stream 1 may start its next tile's P V
                    const float m1 = __uint_as_float(ml0), l1 = __uint_as_float(ml1);
                    const float m_all = fmaxf(m_row, m1);
                    const float base = (m_all == -INFINITY) ? 0.f : m_all;
                    const float fa = fast_exp2(m_row - base), fb = fast_exp2(m1 - base);
#pragma unroll
                    for (int e = 0; e < 32; ++e) o[e] = fmaf(o1[e], fb, o[e] * fa);
                    l_row = fmaf(l1, fb, l_row * fa);
                    m_row = m_all;
                }
                ++didx;
            }
            rzone<kTrace>(tp, tracer, 60, 5);   // the tile's (m, l, O) are final
            if constexpr (kTrace) {
                if (dumping && finish) {
                    float* tail = tp.dump + static_cast<int64_t>(tp.dump_blocks) * kDumpBlock;
#pragma unroll
                    for (int e = 0; e < 32; ++e) tail[row * 64 + group * 32 + e] = o[e];
                    if (group == 0) {
                        tail[128 * 64 + row] = m_row;
                        tail[128 * 64 + 128 + row] = l_row;
                    }
                }
            }
            if (finish && real) {
                const float inv = l_row > 0.f ? 1.f / l_row : 0.f;
                uint32_t w[16];
#pragma unroll
                for (int e = 0; e < 16; ++e) w[e] = pack_bf16(o[2 * e] * inv, o[2 * e + 1] * inv);
                // A thread's 64 bytes lie in a row of their own (32 rows per instruction, a line
                // each): 32-byte stores where the row is aligned for them halve the number of
                // instructions, and with it the time the load/store unit spends on the tile
                // (measured: 1,560 clk from the final values to the stores' issue with four
                // 16-byte stores per thread).
#pragma unroll
                for (int c = 0; c < 2; ++c) {
                    const uint32_t part[8] = {w[c * 8], w[c * 8 + 1], w[c * 8 + 2], w[c * 8 + 3], w[c * 8 + 4], w[c * 8 + 5], w[c * 8 + 6], w[c * 8 + 7]};
                    store_32_bytes(og + c * 16, part);
                }
                if (group == 0 && p.lse) {
                    p.lse[k.b * p.ls[0] + k.h * p.ls[1] + (si.q_off + qi) * p.ls[2]] =
                        l_row > 0.f ? kLn2 * (m_row + log2f(l_row)) : -INFINITY;
                }
            }
            rzone<kTrace>(tp, tracer, 60, 1);
            blk += nb;
            ++uidx;
            first_unit = false;
        }
    }

    // Teardown: everyone arrives (all waits above are bounded), then the allocating warp frees
    // tensor memory.
    tc_fence_before();
    __syncthreads();
    if (is_mma && stream == 0) {
        if (*abort_flag) {
            const long long t0 = clock64();
            while (clock64() - t0 < 2000000) {
            }
        }
        tc_fence_after();
        tmem_dealloc(tmem_base, P::kTmemCols * S);
    }
    if (kTrace && tp.trace && is_mma && lane == 0) {   // lane 0 of a stream's MMA warp knows its block count
        const int cta = blockIdx.x * S + stream;
        if (cta < 1024) {
            long long t1;
            unsigned smid;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1));
            asm volatile("mov.u32 %0, %%smid;" : "=r"(smid));
            long long* out = tp.trace + (64 + cta) * 8;
            out[0] = cta_t0;
            out[1] = t1;
            out[2] = smid;
            out[3] = blocks_done;
        }
    }
}

int sm_count() {
    static int sms[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (!sms[dev]) {
        int n = 148;
        cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
        sms[dev] = n;
    }
    return sms[dev];
}

// Environment switch for experiments: KTT_B200_ROW_DUAL = 0 / 1 forces the mode.
int forced_dual() {
    static int v = -2;
    if (v == -2) {
        const char* e = getenv("KTT_B200_ROW_DUAL");
        v = e ? atoi(e) : -1;
    }
    return v;
}

}  // namespace

bool forward_row_takes(const AttnParams& p, const char** why) {
    if (p.d != 64 || p.dv != 64) {
        *why = "the two-stream kernel is built for head dim 64";
        return false;
    }
    return forward_tc5_takes(p, why);
}

int64_t forward_row_workspace(const AttnParams&) { return kRowHeaderBytes; }

int launch_forward_row(const AttnParams& p, void* workspace, int64_t workspace_bytes, cudaStream_t stream) {
    using P = RowPlan;
    const char* why = "";
    const int64_t tq = p.cu_q ? p.total_q : p.sq, tk = p.cu_q ? p.total_k : p.sk;
    const int64_t bq = p.cu_q ? 1 : p.batch;
    int64_t sq[3], sk[3], sv[3];
    if (!operand_layout(p.q, tq, p.heads, bq, p.qs, sq, &why) ||
        !operand_layout(p.k, tk, p.kv_heads, bq, p.ks, sk, &why) ||
        !operand_layout(p.v, tk, p.kv_heads, bq, p.vs, sv, &why)) {
        return fail(KTT_B200_ERR_UNSUPPORTED, "tcgen05 forward: %s", why);
    }
    const DimOrder orders[3] = {order_of(sq), order_of(sk), order_of(sv)};
    CUtensorMap mq, mk, mv;
    if (!encode_map(&mq, p.q, 64, tq, p.heads, bq, sq, orders[0], kBM, &why) ||
        !encode_map(&mk, p.k, 64, tk, p.kv_heads, bq, sk, orders[1], kBN, &why) ||
        !encode_map(&mv, p.v, 64, tk, p.kv_heads, bq, sv, orders[2], kBN, &why)) {
        return fail(KTT_B200_ERR_UNSUPPORTED, "tcgen05 forward: %s", why);
    }
    RowParams tp;
    tp.a = p;
    int* dev_status = nullptr;
    int* host_status = status_word(&dev_status);
    if (!host_status || !dev_status) return fail(KTT_B200_ERR_LAUNCH, "tcgen05 forward: no status word");
    if (*host_status != 0) {
        const int code = *host_status;
        *host_status = 0;
        note_call(5);
        return fail(KTT_B200_ERR_DEVICE_WAIT, "an earlier tcgen05 launch gave up waiting (code %d)", code);
    }
    tp.status = dev_status;
    tp.trace = tc5::trace_buffer();
    const DumpRequest dump = get_dump_request();
    tp.dump = dump.buffer;
    tp.dump_b = dump.batch;
    tp.dump_h = dump.head;
    tp.dump_q0 = dump.q_tile * kBM;
    tp.dump_blocks = dump.max_blocks;
    for (int o = 0; o < 3; ++o) {
        for (int i = 0; i < 3; ++i) tp.dim_of[o][i] = orders[o].slot_of[i];
    }
    tp.q_tiles = (p.sq + kBM - 1) / kBM;
    tp.by_heads = divisor_of(p.heads);
    tp.by_batch = divisor_of(p.batch > 0 ? p.batch : 1);
    tp.by_kv_heads = divisor_of(p.kv_heads);
    tp.by_group = divisor_of(p.heads / p.kv_heads);
    tp.by_per_pair = divisor_of(tp.q_tiles > 0 ? tp.q_tiles * (p.heads / p.kv_heads) : 1);
    const int64_t tiles = static_cast<int64_t>(p.heads) * p.batch * tp.q_tiles;
    if (tiles > 0x3fffffff) return fail(KTT_B200_ERR_UNSUPPORTED, "tcgen05 forward: too many query tiles");
    tp.units = static_cast<int>(tiles);
    const int sms = sm_count();
    // Few tiles per SM: the two streams of a CTA share each tile.
    tp.dual = tiles <= 6 * static_cast<int64_t>(sms) ? 1 : 0;
    if (forced_dual() >= 0) tp.dual = forced_dual() ? 1 : 0;
    // The counter pays when a dealing position gets several tiles; with one or two the fixed
    // deal (longest first, snake order) is as even and saves the round trip to the counter
    // before each tile's first load.
    const int64_t positions = static_cast<int64_t>(sms) * (tp.dual ? 1 : P::kStreams);
    const bool have_ws = workspace && workspace_bytes >= kRowHeaderBytes && (reinterpret_cast<uintptr_t>(workspace) & 15) == 0 &&
                         tiles > 2 * positions;
    tp.work_counter = have_ws ? static_cast<int*>(workspace) : nullptr;
    tp.done_counter = have_ws ? static_cast<int*>(workspace) + 1 : nullptr;
    // K / V well beyond what L2 keeps (126 MB on B200): the grouped order, which needs the
    // counter. Measured on B x 16 heads x S 8192: 134 MB of K / V 670 (grouped) against 718
    // TFLOP/s, 268 MB 710 against 621, 537 MB 669 against 522.
    const int64_t kv_rows = p.cu_q ? p.total_k : static_cast<int64_t>(p.batch) * p.sk;
    tp.grouped = (have_ws && !tp.dual && kv_rows * p.kv_heads * (p.d + p.dv) * 2 > (192ll << 20)) ? 1 : 0;
    const bool masked = p.mask_dtype != KTT_B200_MASK_NONE;
    const bool traced = tp.trace || tp.dump;
    auto kernel = masked ? (traced ? fwd_row_kernel<true, true> : fwd_row_kernel<false, true>)
                         : (traced ? fwd_row_kernel<true, false> : fwd_row_kernel<false, false>);
    if (int rc = ensure_smem(kernel, P::kBytes, "cudaFuncSetAttribute(fwd_row)")) return rc;
    const int lanes = tp.dual ? 1 : P::kStreams;
    const int64_t want = (tiles + lanes - 1) / lanes;
    const int grid = want < sms ? static_cast<int>(want) : sms;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(grid));
    cfg.blockDim = dim3(P::kThreads);
    cfg.dynamicSmemBytes = P::kBytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return check_cuda(cudaLaunchKernelEx(&cfg, kernel, mq, mk, mv, tp), "fwd_row launch");
}

namespace {
DumpRequest g_dump = {nullptr, 0, 0, 0, 0};
}
void set_dump_request(const DumpRequest& r) { g_dump = r; }
DumpRequest get_dump_request() { return g_dump; }

// Streams (independent query tiles in flight) of the head-dim-64 forward kernel per SM of
// the current device: 2 when a CTA fits.
int forward_row_occupancy() {
    using P = RowPlan;
    auto kernel = fwd_row_kernel<false, false>;
    if (ensure_smem(kernel, P::kBytes, "cudaFuncSetAttribute(fwd_row)")) return -1;
    int n = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kernel, P::kThreads, P::kBytes) != cudaSuccess) return -1;
    return n * P::kStreams;
}

}  // namespace ktt
