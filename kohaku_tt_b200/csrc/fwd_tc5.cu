// Prefill / training forward on the Blackwell tensor path: TMA tile loads, tcgen05.mma
// with accumulators in tensor memory, online softmax in registers.
//
// A persistent CTA per SM walks a list of work items; one item = 128 query rows of one
// (batch, head) against its visible 128-key blocks. Ten warps:
//
//   warp 9 (producer)  TMA loads of an item's Q and of its K/V blocks into a ring of stages
//                      (128-byte swizzled tiles, mbarrier transaction counts); with a work
//                      counter it also draws the items and hands them to the other roles
//   warp 8 (MMA)       issues  S = Q K^T  (128 x 128 x D, both operands K-major from shared
//                      memory) into one of two score buffers in tensor memory, two blocks
//                      ahead of the softmax, and  O_g += P_g V  per softmax group, with P
//                      read from tensor memory and V as the MN-major operand
//   warps 0-3, 4-7     two softmax groups: thread r of group g owns query row r and keys
//                      [64 g, 64 g + 64) of every block, with its own running maximum, sum
//                      and accumulator O_g; it writes P (bf16) over the score columns it
//                      read and rescales O_g only when the maximum moved by more than 2^8
//                      (the lazy rescale of ktt_flash/compute.cpp, flash.md "row
//                      reference"); the groups are merged once per item
//
// Optional per call: a mask of one row per (batch, head), per-batch key lengths, profiling
// stamps (template flags and runtime checks below).
//
// Same arithmetic contract as the reference's flash forward (ktt_flash/compute.cpp:
// 193-491): base-2 softmax with fp32 statistics, P rounded to bf16 before P V, fp32
// accumulation, O / l and lse = ln2 (m + log2 l) at the end.
//
// Every wait on an mbarrier is bounded: when one runs out the CTA records a code in a
// host-visible status word, stops waiting everywhere, frees its tensor memory and exits.
#include <cstring>
#include <mutex>

#include "tc5.cuh"

#include <type_traits>

namespace ktt {
using namespace tc5;
namespace {

constexpr int kTmemCols = 512;    // two S / P buffers, one O accumulator per softmax group
constexpr float kRescaleGap = 8.f;  // in log2 units

// ---- shared-memory plan -----------------------------------------------------------------

// Persistent kernel: one CTA per SM walks a list of work items (128 query rows of one
// (batch, head) each), ten warps:
//   warps 0-3  softmax group a: thread r owns row r and each block's keys [0, 64)
//   warps 4-7  softmax group b: thread r owns row r and each block's keys [64, 128)
//   warp 8     MMA issuer, warp 9 TMA producer
// Each group keeps its own running maximum, sum and output accumulator (O_a, O_b), so the
// two threads of a row never talk inside the loop; the halves are merged once per item.
// While the softmax groups write an item's output, the producer already loads the next
// item's Q / K / V and the MMA warp issues its first two Q K^T: barriers, the K/V ring and
// tensor memory live across items.
// Tensor memory (512 columns): S / P buffers [0, 128) and [128, 256) (P overwrites the S
// columns it came from as packed bf16), O_a [256, 256 + D), O_b [256 + D, 256 + 2 D).
template <int D>
struct Plan {
    // Softmax groups: each owns 128 / kGroups of a block's keys and its own accumulator.
    // (Four groups were tried at D 64 with the registers re-divided by setmaxnreg: the
    // softmax loop is bound by the SM's MUFU / FMA / issue rates, not by latency, and
    // sixteen warps ran no faster than eight.)
    static constexpr int kGroups = 2;
    // Pairs of exponentials per thread and block that take the FMA-pipe polynomial instead
    // of MUFU. Measured: 4 of 32 is best by ~2 %; more loses to the extra instructions.
    static constexpr int kPolyPairs = 4;
    static constexpr int kCols = 128 / kGroups;          // score columns per softmax thread
    static constexpr int kThreads = 128 * kGroups + 64;  // softmax warps + MMA warp + producer warp
    static constexpr int kMmaWarp = 4 * kGroups;
    static constexpr int kSub = D / 64;                  // 64-column sub-tiles of Q, K, V
    static constexpr int kTile = 128 * 128;              // one [128][64] bf16 sub-tile
    static constexpr int kStages = D == 64 ? 4 : 3;      // K/V ring depth
    static constexpr int kQ = 0;
    static constexpr int kK = kQ + kSub * kTile;
    static constexpr int kV = kK + kStages * kSub * kTile;
    static constexpr int kML = kV + kStages * kSub * kTile;   // float2 [groups][128]: (m, l)
    static constexpr int kMaskRow = kML + kGroups * 128 * 8;   // float [groups][128 / groups]: a block's mask terms
    static constexpr int kBars = kMaskRow + 128 * 4;
    static constexpr int kBarBytes = 384;
    static constexpr int kBytes = kBars + kBarBytes;
    static_assert(kBytes <= 232448, "shared memory per CTA");
    // barrier indices (8 bytes each)
    static constexpr int bQFull = 0;
    static constexpr int bQFree = 1;
    static constexpr int bOFree = 2;
    static constexpr int bKVFull = 3;                 // + stage
    static constexpr int bKVEmpty = bKVFull + kStages;
    static constexpr int bSFull = bKVEmpty + kStages;  // + buffer
    // P published / P V complete: one barrier per (group, S buffer). A parity wait tells
    // phases apart only one step deep, and a group may run two blocks ahead of the MMA warp
    // (or the MMA warp two P V ahead of a group's next look); alternating barriers keeps
    // every one of them within one phase of its waiters.
    static constexpr int bPFull = bSFull + 2;              // + 2 * group + buffer
    static constexpr int bPVDone = bPFull + 2 * kGroups;   // + 2 * group + buffer
    static constexpr int bMaskRow = bPVDone + 2 * kGroups; // + 2 * group + (0: readers done, 1: row written)
    static constexpr int bWorkFull = bMaskRow + 2 * kGroups;   // + slot: an item index was published
    static constexpr int bWorkFree = bWorkFull + 2;            // + slot: every reader has taken it
    static constexpr int bEpilogue = bWorkFree + 2;            // all softmax threads have stored (m, l) of the item
    static constexpr int bCount = bEpilogue + 1;
    static_assert(bCount * 8 + 16 + 4 * kMmaWarp + 16 <= kBarBytes, "barrier area");
    static_assert(256 + kGroups * D <= 512, "tensor memory columns");
};

struct Tc5Params {
    AttnParams a;
    int* status;        // host-visible: first wait that ran out, or 0
    int dim_of[3][3];   // per operand (q, k, v): tensor-map coordinate slot (1..3) of the
                        // row, head and batch dims
    long long* trace;   // optional clock stamps (see ktt_b200_set_trace), else null
    int q_tiles;        // query tiles per batch entry (ceil(sq / 128))
    int work;           // work items = heads * batch * q_tiles
    int* work_counter;  // optional (zero before the launch): the CTAs draw their items from it
    int* done_counter;  // with it: producers that have drawn their last; the last one puts both back to zero
    int grouped;        // item order (decode_work): 1 with a counter
    Divisor by_heads, by_batch, by_kv_heads, by_group, by_per_pair;   // group: query heads per K/V head; per_pair: q_tiles * group
};

// Profiling zones (the counterpart of the reference's FLASH_PROFILE device zones,
// ktt_flash/compute.cpp:25-30): CTA 0 stamps clock64 per key block of its first item.
//   slots 0-3: softmax row 0 of group a after S ready / maximum known / exponentials done /
//              P published;  slot 4: MMA lane before the next-but-one Q K^T;
//   slots 5-7: MMA lane after issuing P V of half a / of half b / the next-but-one Q K^T.
// The stamps cost a few percent even when nobody listens, so the traced kernel is an
// instantiation of its own, launched only while a trace buffer is set.
template <bool kTrace>
__device__ __forceinline__ void zone(const Tc5Params& tp, bool who, int j, int slot) {
    if constexpr (kTrace) {
        if (who && j < 64) tp.trace[j * 8 + slot] = clock64();
    }
}

// One work item: 128 query rows of (batch b, head h).
struct Work {
    int b, h, q0, nblocks;
    SeqInfo si;
    bool valid;  // false: the tile lies past the end of its sequence
};

// Two orders of the items. Fixed deal (no counter): consecutive items are the heads of one
// (tile, batch) and the longest causal tiles come first, so that the snake deal below gives
// every CTA a similar mix of long and short tiles. Drawn from a counter (`grouped`): all
// query tiles of one (batch, K/V head) follow one another, longest first, the heads of the
// GQA group fastest: the ~148 tiles in flight at any time then read the K / V of a handful
// of (batch, head) pairs, which stay in L2, instead of one tile of every pair in the launch
// (measured on the packed 65,536-token batch, 537 MB of K / V: 4.85 GB of DRAM reads per
// launch for 1.07 GB of operands with the first order). The counter keeps the load even.
__device__ __forceinline__ Work decode_work(const Tc5Params& tp, int w) {
    const AttnParams& p = tp.a;
    Work k;
    int qb;
    if (tp.grouped) {
        const int group = static_cast<int>(tp.by_group.d);
        const int pair = div_by(w, tp.by_per_pair), r = w - pair * static_cast<int>(tp.by_per_pair.d);
        const int tile = div_by(r, tp.by_group);
        k.b = div_by(pair, tp.by_kv_heads);
        k.h = (pair - k.b * p.kv_heads) * group + (r - tile * group);
        qb = tp.q_tiles - 1 - tile;
    } else {
        const int t = div_by(w, tp.by_heads), level = div_by(t, tp.by_batch);
        k.h = w - t * p.heads;
        k.b = t - level * p.batch;
        qb = tp.q_tiles - 1 - level;
    }
    k.si = seq_info(p, k.b);
    k.q0 = qb * kBM;
    k.valid = k.q0 < k.si.lq;
    int kend = k.si.klen;
    if (p.causal) kend = min(kend, min(k.q0 + kBM, k.si.lq) - 1 + k.si.shift + 1);
    k.nblocks = (k.valid && kend > 0) ? (kend + kBN - 1) / kBN : 0;
    return k;
}

// Items are dealt to the CTAs in snake order (0 .. G-1, then G-1 .. 0, ...): on a list
// sorted by decreasing work that pairs each CTA's long items with short ones.
__device__ __forceinline__ int work_of(int round, int cta, int ctas) {
    return round * ctas + ((round & 1) ? ctas - 1 - cta : cta);
}

// ---- the kernel ------------------------------------------------------------------------

template <int D, bool kTrace, bool kMask>
__global__ void __launch_bounds__(Plan<D>::kThreads, 1) fwd_tc5_kernel(
    const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
    const __grid_constant__ CUtensorMap map_v, const Tc5Params tp) {
    using P = Plan<D>;
    constexpr int G = P::kGroups, CG = P::kCols;
    constexpr int kSoftmaxThreads = 128 * G;
    extern __shared__ __align__(1024) unsigned char smem[];
    const uint32_t sbase = smem_u32(smem);
    // Swizzled tiles need a 1024-byte aligned base. The dynamic window starts there on
    // every launch seen so far; refuse to run rather than compute garbage if it does not.
    if (sbase & 1023u) {
        if (threadIdx.x == 0) atomicCAS_system(tp.status, 0, 900);
        return;
    }
    // Second profiling zone set: rows 64.. of the trace buffer hold, per CTA, its start and
    // end on the global nanosecond timer, its SM and the key blocks it processed.
    long long cta_t0 = 0;
    long long cta_c0 = 0;
    if (kTrace && threadIdx.x == kSoftmaxThreads) {
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(cta_t0));
        cta_c0 = clock64();
    }
    const uint32_t bars = sbase + P::kBars;
    auto bar = [&](int i) { return bars + 8u * i; };
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + P::kBars + P::bCount * 8);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + P::kBars + P::bCount * 8 + 8);
    // Per item and softmax warp: "every wait of mine succeeded" (two items alternate).
    volatile int* ok_flags = reinterpret_cast<volatile int*>(smem + P::kBars + P::bCount * 8 + 16);
    volatile int* work_slot = ok_flags + P::kMmaWarp;       // [2] item indices drawn from the counter (after one flag per softmax warp)

    const AttnParams& p = tp.a;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    // The producer warp sets the barriers up itself and goes straight to its first loads;
    // it only arrives at the start-up barrier, the others wait there for it and for the
    // tensor-memory allocation.
    if (warp == P::kMmaWarp + 1) {
      // One barrier per lane: lane i initialises barrier i with its arrival count.
      static_assert(P::bCount <= 32, "one barrier per lane");
      if (lane < P::bCount) {
        uint32_t count = 1;
        // Softmax threads arrive once per warp (mbar_arrive_warp).
        if (lane == P::bOFree) count = 4 * G;
        if ((lane >= P::bPFull && lane < P::bPVDone) || (lane >= P::bMaskRow && lane < P::bWorkFull)) count = 4;
        if (lane >= P::bWorkFree) count = 4 * G + 1;   // every softmax warp and the MMA warp
        if (lane == P::bEpilogue) count = 4 * G;
        mbar_init(bar(lane), count);
      }
      if (lane == 0) {
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_q) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_k) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_v) : "memory");
        *abort_flag = 0;
      }
      asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
      fence_async_smem();
      __syncwarp();
      asm volatile("barrier.cta.arrive 0, %0;" ::"n"(P::kThreads) : "memory");
    } else {
      if (warp == P::kMmaWarp) tmem_alloc(smem_u32(tmem_slot), kTmemCols);
      tc_fence_before();
      asm volatile("barrier.cta.sync 0, %0;" ::"n"(P::kThreads) : "memory");
      tc_fence_after();
    }
    const uint32_t tmem = *tmem_slot;
    const uint32_t tmem_o = tmem + 256;    // one accumulator of D columns per group

    // Tensor-map coordinates: slot 0 is the head dim; rows, head and batch sit in the
    // slots the host sorted them into by stride.
    auto coords = [&](int operand, int row, int head, int batch, int (&c)[4]) {
        c[tp.dim_of[operand][0]] = row;
        c[tp.dim_of[operand][1]] = head;
        c[tp.dim_of[operand][2]] = batch;
    };

    // Every role walks the same items and keeps the same two counters: `item` counts the
    // items with at least one key block, `blk` the key blocks of all items so far. Ring
    // stages, S buffers and barrier parities are functions of those.
    int blocks_done = 0;

    // The n-th item of this CTA: -1 = no more, -2 = nothing at this position. Without a
    // counter every role computes the same snake order by itself. With one, the producer
    // warp draws indices (the list is sorted by decreasing work, so a CTA that started late
    // or shares its SM simply draws fewer) and hands each to the other roles through a
    // two-slot queue in shared memory.
    const bool dynamic = tp.work_counter != nullptr;
    auto static_item = [&](int n) -> int {
        if (static_cast<int64_t>(n) * gridDim.x >= tp.work) return -1;
        const int w = work_of(n, blockIdx.x, gridDim.x);
        return w < tp.work ? w : -2;
    };
    auto draw_item = [&](int n, bool& ok) -> int {   // producer warp, converged
        if (!dynamic) return static_item(n);
        const int slot = n & 1;
        if (n >= 2) {
            ok = __all_sync(0xffffffffu, mbar_wait(bar(P::bWorkFree + slot), ((n >> 1) - 1) & 1, abort_flag, 120 + slot, tp.status));
            if (!ok) return -1;
        }
        // Positions past the end of their sequence (packed batches have many) are skipped
        // here, so the other roles never see them.
        int w;
        while (true) {
            w = 0;
            if (lane == 0) w = atomicAdd(tp.work_counter, 1);
            w = __shfl_sync(0xffffffffu, w, 0);
            if (w >= tp.work) {
                w = -1;
                break;
            }
            if (decode_work(tp, w).valid) break;
        }
        if (lane == 0) {
            work_slot[slot] = w;
            __threadfence_block();
            mbar_arrive(bar(P::bWorkFull + slot));
        }
        return w;
    };
    auto take_item = [&](int n, bool& ok, bool arrives) -> int {   // the other roles
        if (!dynamic) return static_item(n);
        const int slot = n & 1;
        ok = __all_sync(0xffffffffu, mbar_wait(bar(P::bWorkFull + slot), (n >> 1) & 1, abort_flag, 130 + slot, tp.status));
        if (!ok) return -1;
        const int w = work_slot[slot];
        if (arrives) mbar_arrive_warp(bar(P::bWorkFree + slot));
        return w;
    };

    if (warp == P::kMmaWarp + 1) {
        // ---------------- producer (whole warp, converged) ----------------
        int item = 0, blk = 0;
        bool ok = true;
        // Drawn items are fetched one ahead: the trip to the counter (and the positions past
        // the end of short sequences that a draw skips) then hides behind a whole item's loads
        // instead of standing between two items.
        int w_next = draw_item(0, ok);
        for (int n = 0; ok; ++n) {
            const int w = w_next;
            if (w == -1) break;
            w_next = draw_item(n + 1, ok);
            if (!ok) break;
            if (w == -2) continue;
            const Work k = decode_work(tp, w);
            if (k.nblocks == 0) continue;
            const int hk = div_by(k.h, tp.by_group);
            int c[4], cv[4];
            const int batch = p.cu_q ? 0 : k.b;
            c[0] = cv[0] = 0;
            // Q may be replaced once the last Q K^T of the previous item has run.
            if (item > 0) {
                ok = __all_sync(0xffffffffu, mbar_wait(bar(P::bQFree), (item - 1) & 1, abort_flag, 110, tp.status));
                if (!ok) break;
            }
            coords(0, k.si.q_off + k.q0, k.h, batch, c);
            mbar_expect_tx(bar(P::bQFull), P::kSub * P::kTile);
            for (int s = 0; s < P::kSub; ++s) {
                tma_load_4d(sbase + P::kQ + s * P::kTile, &map_q, bar(P::bQFull), s * 64, c[1], c[2], c[3]);
            }
            for (int j = 0; j < k.nblocks; ++j) {
                const int gb = blk + j, st = gb % P::kStages;
                if (gb >= P::kStages) {
                    ok = __all_sync(0xffffffffu, mbar_wait(bar(P::bKVEmpty + st), ((gb / P::kStages) - 1) & 1, abort_flag, 100 + st, tp.status));
                    if (!ok) break;
                }
                coords(1, k.si.k_off + j * kBN, hk, batch, c);
                coords(2, k.si.k_off + j * kBN, hk, batch, cv);
                mbar_expect_tx(bar(P::bKVFull + st), 2 * P::kSub * P::kTile);
                for (int s = 0; s < P::kSub; ++s) {
                    tma_load_4d(sbase + P::kK + (st * P::kSub + s) * P::kTile, &map_k, bar(P::bKVFull + st), s * 64, c[1], c[2], c[3]);
                    tma_load_4d(sbase + P::kV + (st * P::kSub + s) * P::kTile, &map_v, bar(P::bKVFull + st), s * 64, cv[1], cv[2], cv[3]);
                }
            }
            blk += k.nblocks;
            ++item;
        }
        if (*abort_flag) {
            // Let copies already in flight land before the CTA's memory goes away.
            const long long t0 = clock64();
            while (clock64() - t0 < 4000000) {
            }
        } else if (dynamic && tp.done_counter && lane == 0) {
            // This producer draws no more. The last one to say so puts the counters back to
            // zero for the next launch.
            __threadfence();
            const int done = atomicAdd(tp.done_counter, 1);
            if (done == static_cast<int>(gridDim.x) - 1) {
                *tp.work_counter = 0;
                *tp.done_counter = 0;
                __threadfence();
            }
        }
    } else if (warp == P::kMmaWarp) {
        // ---------------- MMA issuer (whole warp, converged) ----------------
        constexpr uint32_t idesc_s = instr_desc(kBN, false);
        constexpr uint32_t idesc_o = instr_desc(D, true);
        // Descriptors differ only in their 14-bit start-address field (bytes / 16):
        // build each base once and add constants per MMA.
        const uint64_t q_desc = smem_desc(sbase + P::kQ, 16, 1024);
        const uint64_t k_desc = smem_desc(sbase + P::kK, 16, 1024);
        const uint64_t v_desc = smem_desc(sbase + P::kV, P::kTile, 1024);
        int item = 0, blk = 0;
        bool ok = true;
        bool first_item = true;
        // Q K^T of global block gb into S buffer gb & 1; `last` marks the item's last one,
        // after which Q is free.
        auto issue_s = [&](int gb, bool last) {
            const uint64_t kd = k_desc + static_cast<uint64_t>(((gb % P::kStages) * P::kSub * P::kTile) >> 4);
            const uint32_t d_s = tmem + (gb & 1) * 128;
#pragma unroll
            for (int ks = 0; ks < D / 16; ++ks) {
                const uint32_t off = ((ks / 4) * P::kTile + (ks % 4) * 32) >> 4;
                tc_mma(d_s, q_desc + off, kd + off, idesc_s, ks > 0);
            }
            tc_commit(bar(P::bSFull + (gb & 1)));
            if (last) tc_commit(bar(P::bQFree));
        };
        for (int n = 0; ok; ++n) {
            const int w = take_item(n, ok, true);
            if (w == -1) break;
            if (w == -2) continue;
            const Work k = decode_work(tp, w);
            if (k.nblocks == 0) continue;
            const bool mtracer = first_item && lane == 0 && blockIdx.x == 0;
            zone<kTrace>(tp, mtracer, 61, 0);
            ok = __all_sync(0xffffffffu, mbar_wait(bar(P::bQFull), item & 1, abort_flag, 200, tp.status));
            zone<kTrace>(tp, mtracer, 61, 1);
            // The first two Q K^T of the item run while the previous item's output is
            // still being written: they only need the S buffers, which are free once the
            // previous item's P V MMAs have been issued.
            for (int j = 0; ok && j < 2 && j < k.nblocks; ++j) {
                const int gb = blk + j;
                ok = __all_sync(0xffffffffu, mbar_wait(bar(P::bKVFull + gb % P::kStages), (gb / P::kStages) & 1, abort_flag, 210 + j, tp.status));
                if (ok) {
                    tc_fence_after();
                    zone<kTrace>(tp, mtracer, 61, 2 + j);
                    issue_s(gb, j + 1 == k.nblocks);
                }
            }
            for (int j = 0; ok && j < k.nblocks; ++j) {
                const int gb = blk + j, st = gb % P::kStages;
                const uint64_t vd = v_desc + static_cast<uint64_t>((st * P::kSub * P::kTile) >> 4);
                const uint32_t p_tmem = tmem + (gb & 1) * 128;
                if (j == 0 && item > 0) {
                    // The accumulators are free once the previous item's epilogue has read them.
                    ok = __all_sync(0xffffffffu, mbar_wait(bar(P::bOFree), (item - 1) & 1, abort_flag, 250, tp.status));
                    if (!ok) break;
                }
                if (p.key_lengths) {
                    // Rows of the cache past this sequence's length may hold anything, and
                    // P = 0 times an infinity would still poison the output: the value rows
                    // past the length are blanked in the tile before P V reads it (TMA itself
                    // only blanks rows past the end of the tensor). The key rows need nothing:
                    // their scores are replaced before use.
                    const int valid = k.si.klen - j * kBN;
                    if (valid < kBN) {
                        const int rows = kBN - (valid > 0 ? valid : 0), first = kBN - rows;
                        unsigned char* vt = smem + P::kV + st * P::kSub * P::kTile;
                        for (int idx = lane; idx < P::kSub * rows * 8; idx += 32) {
                            const int sub = idx / (rows * 8), rem = idx % (rows * 8);
                            *reinterpret_cast<uint4*>(vt + sub * P::kTile + (first + rem / 8) * 128 + (rem % 8) * 16) =
                                make_uint4(0u, 0u, 0u, 0u);
                        }
                        fence_async_smem();
                        __syncwarp();
                    }
                }
#pragma unroll
                for (int g = 0; g < G; ++g) {
                    ok = __all_sync(0xffffffffu, mbar_wait(bar(P::bPFull + 2 * g + (gb & 1)), (gb >> 1) & 1, abort_flag, 240 + g, tp.status));
                    if (!ok) break;
                    tc_fence_after();
#pragma unroll
                    for (int ks = 0; ks < CG / 16; ++ks) {
                        // A: this group's P, 8 TMEM columns per 16 keys. B: V is MN-major, 16
                        // keys down = 16 rows of 128 bytes; the second 64 columns of D are
                        // one sub-tile further (LBO).
                        tc_mma_ts(tmem_o + g * D, p_tmem + g * CG + ks * 8,
                                  vd + (((g * (CG / 16) + ks) * 2048) >> 4), idesc_o, (j > 0 || ks > 0) ? 1u : 0u);
                    }
                    tc_commit(bar(P::bPVDone + 2 * g + (gb & 1)));
                    if (g < 2) zone<kTrace>(tp, mtracer, j, 5 + g);
                }
                if (!ok) break;
                tc_commit(bar(P::bKVEmpty + st));
                if (j + 2 < k.nblocks) {
                    // Both groups have published P of block j, so they are done with this S
                    // buffer; MMAs run in issue order, so the P V reads above precede the
                    // overwrite.
                    const int gb2 = gb + 2;
                    ok = __all_sync(0xffffffffu, mbar_wait(bar(P::bKVFull + gb2 % P::kStages), (gb2 / P::kStages) & 1, abort_flag, 220, tp.status));
                    if (!ok) break;
                    tc_fence_after();
                    zone<kTrace>(tp, mtracer, j, 4);
                    issue_s(gb2, j + 3 == k.nblocks);
                    zone<kTrace>(tp, mtracer, j, 7);
                }
            }
            blk += k.nblocks;
            ++item;
            first_item = false;
        }
        blocks_done = blk;
    } else {
        // ---------------- softmax: thread = (query row, half of each block's keys) ----------------
        const int g = warp >> 2;                        // group: keys [g * CG, (g + 1) * CG) of each block
        const int row = (warp & 3) * 32 + lane;         // row inside the tile = TMEM lane
        const uint32_t lane_addr = static_cast<uint32_t>((warp & 3) * 32) << 16;
        int item = 0, blk = 0;
        bool ok = true;
        bool first_item = true;
        float2* ml_base = reinterpret_cast<float2*>(smem + P::kML);

        for (int n = 0; ok; ++n) {
            const int w = take_item(n, ok, true);
            if (w == -1) break;
            if (w == -2) continue;
            const Work k = decode_work(tp, w);
            if (!k.valid) continue;
            const SeqInfo& si = k.si;
            const int qi = k.q0 + row;                  // row inside the sequence
            const bool real = qi < si.lq;
            __nv_bfloat16* og = p.out + k.b * p.os[0] + k.h * p.os[1] + static_cast<int64_t>(si.q_off + qi) * p.os[2] + g * (D / G);
            if (k.nblocks == 0) {
                // No key is visible to this tile: zeros, lse = -inf. No barrier is involved.
                if (real) {
#pragma unroll
                    for (int c = 0; c < D / G / 8; ++c) *reinterpret_cast<uint4*>(og + c * 8) = make_uint4(0u, 0u, 0u, 0u);
                    if (g == 0 && p.lse) p.lse[k.b * p.ls[0] + k.h * p.ls[1] + (si.q_off + qi) * p.ls[2]] = -INFINITY;
                }
                continue;
            }
            const bool tracer = first_item && row == 0 && blockIdx.x == 0;
            float m_ref = -INFINITY;  // this half's reference maximum (base-2 logits), moved lazily
            float2 l2[2] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f)};  // running sums, 4 lanes
            // Keys this row may see: [0, row_limit).
            int row_limit = si.klen;
            if (p.causal) row_limit = min(row_limit, qi + si.shift + 1);

            for (int j = 0; ok && j < k.nblocks; ++j) {
                const int gb = blk + j;
                const uint32_t s_addr = tmem + (gb & 1) * 128 + g * CG + lane_addr;
                ok = __all_sync(0xffffffffu, mbar_wait(bar(P::bSFull + (gb & 1)), (gb >> 1) & 1, abort_flag, 300 + g, tp.status));
                if (!ok) break;
                tc_fence_after();
                zone<kTrace>(tp, tracer && g == 0, j, 0);
                float s[CG];
                const int limit = row_limit - j * kBN - g * CG;  // this group's columns [0, limit) are visible
                float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
                const bool whole = limit >= CG;
                // With a mask that is one row per (batch, head) the base-2 terms of this
                // group's 64 keys are fetched first (indices clamped, loads unconditional)
                // and are in flight with the scores.
                float mk[kMask ? CG : 1];
                if constexpr (kMask) {
                    // One thread per column fetches the term (index clamped into the
                    // sequence), the group shares the row through shared memory. The first
                    // barrier keeps the previous block's readers ahead of the writers.
                    // (Group-wide mbarriers with bounded waits, not bar.sync: a warp that has
                    // given up elsewhere must not leave the others waiting here for ever.)
                    float* mrow = reinterpret_cast<float*>(smem + P::kMaskRow) + g * CG;
                    mbar_arrive_warp(bar(P::bMaskRow + 2 * g));
                    ok = __all_sync(0xffffffffu, mbar_wait(bar(P::bMaskRow + 2 * g), gb & 1, abort_flag, 340 + g, tp.status));
                    if (!ok) break;
                    if (row < CG) {
                        const int jj = max(min(j * kBN + g * CG + row, si.klen - 1), 0);
                        mrow[row] = mask_value(p, k.b, k.h, 0, static_cast<int64_t>(si.k_off) + jj) * kLog2e;
                    }
                    mbar_arrive_warp(bar(P::bMaskRow + 2 * g + 1));
                    ok = __all_sync(0xffffffffu, mbar_wait(bar(P::bMaskRow + 2 * g + 1), gb & 1, abort_flag, 350 + g, tp.status));
                    if (!ok) break;
#pragma unroll
                    for (int e4 = 0; e4 < CG / 4; ++e4) {
                        const float4 t = reinterpret_cast<const float4*>(mrow)[e4];
                        mk[e4 * 4] = t.x; mk[e4 * 4 + 1] = t.y; mk[e4 * 4 + 2] = t.z; mk[e4 * 4 + 3] = t.w;
                    }
                }
                // The second half of the columns is still on its way while the maximum of
                // the first is taken.
                tmem_ld32(s_addr, s);
                tmem_wait_ld();
                tmem_ld32(s_addr + 32, s + 32);
                if constexpr (kMask) {
                    // Logits in place: s * scale + mask term; the maximum is taken over those.
#pragma unroll
                    for (int e = 0; e < 32; ++e) s[e] = fmaf(s[e], p.scale_log2, mk[e]);
                }
                if (whole) {
#pragma unroll
                    for (int e = 0; e < 32; ++e) mx4[e & 3] = fmaxf(mx4[e & 3], s[e]);
                }
                tmem_wait_ld();
                if constexpr (kMask) {
#pragma unroll
                    for (int e = 32; e < CG; ++e) s[e] = fmaf(s[e], p.scale_log2, mk[e]);
                }
                if (whole) {
#pragma unroll
                    for (int e = 32; e < CG; ++e) mx4[e & 3] = fmaxf(mx4[e & 3], s[e]);
                } else {
#pragma unroll
                    for (int e = 0; e < CG; ++e) {
                        s[e] = e < limit ? s[e] : -INFINITY;
                        mx4[e & 3] = fmaxf(mx4[e & 3], s[e]);
                    }
                }
                const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * (kMask ? 1.f : p.scale_log2);
                zone<kTrace>(tp, tracer && g == 0, j, 1);

                // Lazy rescale: move the reference only when this block exceeds it by 2^8.
                const bool move = mx > m_ref + kRescaleGap;
                if (__any_sync(0xffffffffu, move)) {
                    float f = 1.f;
                    if (move) {
                        f = fast_exp2(m_ref - mx);  // 0 on the first block
                        m_ref = mx;
                        l2[0] = __fmul2_rn(l2[0], make_float2(f, f));
                        l2[1] = __fmul2_rn(l2[1], make_float2(f, f));
                    }
                    if (j > 0) {
                        // O of this half holds blocks [0, j): wait for block j - 1's P V.
                        ok = __all_sync(0xffffffffu, mbar_wait(bar(P::bPVDone + 2 * g + ((gb - 1) & 1)), ((gb - 1) >> 1) & 1, abort_flag, 310 + g, tp.status));
                        if (!ok) break;
                        tc_fence_after();
                        // One chunk at a time keeps this rare path from claiming registers.
                        constexpr int kR = 32;
#pragma unroll 1
                        for (int c = 0; c < D / kR; ++c) {
                            float o[kR];
                            const uint32_t addr = tmem_o + g * D + lane_addr + c * kR;
                            if constexpr (kR == 32) {
                                tmem_ld32(addr, o);
                            } else {
                                tmem_ld16(addr, o);
                            }
                            tmem_wait_ld();
#pragma unroll
                            for (int e = 0; e < kR; ++e) o[e] *= f;
                            if constexpr (kR == 32) {
                                tmem_st32(addr, o);
                            } else {
                                tmem_st16(addr, reinterpret_cast<const uint32_t*>(o));
                            }
                        }
                        tmem_wait_st();
                    }
                }
                const float m_use = (m_ref == -INFINITY) ? 0.f : m_ref;

                // P = 2^(s * scale - m) as packed bf16 pairs, two values per instruction where
                // the packed fp32 pipe allows.
                uint32_t wv[CG / 2];
                const float sc1 = kMask ? 1.f : p.scale_log2;  // masked logits are already scaled
                const float2 sc2 = make_float2(sc1, sc1), nm2 = make_float2(-m_use, -m_use);
                if (whole) {
                    // Every column visible. kPolyPairs of this thread's pairs take the polynomial
                    // on the FMA pipe, the rest MUFU; odd groups start with the polynomial and
                    // even ones end with it, so that the warps sharing a scheduler are on
                    // different pipes at the same time.
                    auto exps = [&](auto poly_first) {
                        constexpr bool kFirst = decltype(poly_first)::value;
#pragma unroll
                        for (int e = 0; e < CG / 2; ++e) {
                            const float2 x = __ffma2_rn(make_float2(s[2 * e], s[2 * e + 1]), sc2, nm2);
                            float2 pr;
                            if (kFirst ? (e < P::kPolyPairs) : (e >= CG / 2 - P::kPolyPairs)) {
                                pr = exp2_poly2(x);
                            } else {
                                pr.x = fast_exp2(x.x);
                                pr.y = fast_exp2(x.y);
                            }
                            l2[e & 1] = __fadd2_rn(l2[e & 1], pr);
                            wv[e] = pack_bf16(pr.x, pr.y);
                        }
                    };
                    if (g & 1) {
                        exps(std::true_type{});
                    } else {
                        exps(std::false_type{});
                    }
                } else {
                    // Masked columns take the MUFU path, whose 2^-inf is exactly 0.
#pragma unroll
                    for (int e = 0; e < CG / 2; ++e) {
                        const float2 x = __ffma2_rn(make_float2(s[2 * e], s[2 * e + 1]), sc2, nm2);
                        const float2 pr = make_float2(fast_exp2(x.x), fast_exp2(x.y));
                        l2[e & 1] = __fadd2_rn(l2[e & 1], pr);
                        wv[e] = pack_bf16(pr.x, pr.y);
                    }
                }
                zone<kTrace>(tp, tracer && g == 0, j, 2);
                // P overwrites the first half of the S columns this thread has just read.
                if constexpr (CG == 64) {
                    tmem_st32(s_addr, reinterpret_cast<const float*>(wv));
                } else {
                    tmem_st16(s_addr, wv);
                }
                tmem_wait_st();
                tc_fence_before();
                mbar_arrive_warp(bar(P::bPFull + 2 * g + (gb & 1)));
                zone<kTrace>(tp, tracer && g == 0, j, 3);
            }

            // Epilogue of the item: merge the two halves of each row and normalise. Every lane
            // takes part in the TMEM reads and in the 256-thread barrier whatever happened.
            const int last = blk + k.nblocks - 1;
            // Each group waits for its own last P V; the barrier below then covers all of them.
            if (ok) ok = __all_sync(0xffffffffu, mbar_wait(bar(P::bPVDone + 2 * g + (last & 1)), (last >> 1) & 1, abort_flag, 330 + g, tp.status));
            // One buffer is enough: nobody reaches the next item's write before every thread has
            // passed this item's accumulator hand-over (bOFree), which comes after its reads here.
            zone<kTrace>(tp, tracer && g == 0, 60, 0);
            float2* ml = ml_base;
            const float l_mine = (l2[0].x + l2[0].y) + (l2[1].x + l2[1].y);
            ml[g * 128 + row] = make_float2(m_ref, l_mine);
            if (lane == 0) ok_flags[warp] = ok;
            // A bounded wait like every other in this kernel: no warp can be left behind at a
            // plain barrier by one that has given up.
            mbar_arrive_warp(bar(P::bEpilogue));
            {
                const bool all_here = __all_sync(0xffffffffu, mbar_wait(bar(P::bEpilogue), item & 1, abort_flag, 360 + g, tp.status));
                ok = ok && all_here;
            }
            zone<kTrace>(tp, tracer && g == 0, 60, 1);
            // All softmax warps take the same decision, so none is left alone at this barrier.
#pragma unroll
            for (int i = 0; i < 4 * G; ++i) ok = ok && ok_flags[i] != 0;
            if (ok) {
                // Merge the groups' (m, l) of this row; f[i] rescales group i's accumulator.
                float m_all = -INFINITY;
                float2 mls[G];
#pragma unroll
                for (int i = 0; i < G; ++i) {
                    mls[i] = ml[i * 128 + row];
                    m_all = fmaxf(m_all, mls[i].x);
                }
                const float base = (m_all == -INFINITY) ? 0.f : m_all;
                float f[G], l_sum = 0.f;
#pragma unroll
                for (int i = 0; i < G; ++i) {
                    f[i] = fast_exp2(mls[i].x - base);
                    l_sum += mls[i].y * f[i];
                }
                const float inv = l_sum > 0.f ? 1.f / l_sum : 0.f;
                // Group g writes output columns [g * D / G, (g + 1) * D / G).
                constexpr int kOut = D / G;                  // columns per thread
                constexpr int kChunk = kOut < 32 ? kOut : 32;
                tc_fence_after();
#pragma unroll
                for (int c = 0; c < kOut / kChunk; ++c) {
                    // All groups' chunks are requested before the one wait.
                    float o[G][kChunk];
#pragma unroll
                    for (int i = 0; i < G; ++i) {
                        const uint32_t addr = tmem_o + i * D + lane_addr + g * kOut + c * kChunk;
                        if constexpr (kChunk == 32) {
                            tmem_ld32(addr, o[i]);
                        } else {
                            tmem_ld16(addr, o[i]);
                        }
                    }
                    tmem_wait_ld();
                    float acc[kChunk];
#pragma unroll
                    for (int e = 0; e < kChunk; ++e) acc[e] = o[0][e] * (f[0] * inv);
#pragma unroll
                    for (int i = 1; i < G; ++i) {
                        const float fi = f[i] * inv;
#pragma unroll
                        for (int e = 0; e < kChunk; ++e) acc[e] = fmaf(o[i][e], fi, acc[e]);
                    }
                    zone<kTrace>(tp, tracer && g == 0, 60, 2);
                    if (c + 1 == kOut / kChunk) {
                        // The accumulators are in registers: the next item's P V may overwrite them.
                        tc_fence_before();
                        mbar_arrive_warp(bar(P::bOFree));
                    }
                    if (real) {
#pragma unroll
                        for (int e = 0; e < kChunk / 16; ++e) {
                            uint32_t w[8];
#pragma unroll
                            for (int i = 0; i < 8; ++i) w[i] = pack_bf16(acc[e * 16 + 2 * i], acc[e * 16 + 2 * i + 1]);
                            store_32_bytes(og + c * kChunk + e * 16, w);
                        }
                    }
                }
                zone<kTrace>(tp, tracer && g == 0, 60, 3);
                if (real && g == 0 && p.lse) {
                    p.lse[k.b * p.ls[0] + k.h * p.ls[1] + (si.q_off + qi) * p.ls[2]] =
                        l_sum > 0.f ? kLn2 * (m_all + log2f(l_sum)) : -INFINITY;
                }
            } else {
                break;
            }
            blk += k.nblocks;
            ++item;
            first_item = false;
        }
    }

    // Teardown: everyone arrives (all waits above are bounded), then the allocating warp
    // frees tensor memory.
    tc_fence_before();
    __syncthreads();
    if (warp == P::kMmaWarp) {
        if (*abort_flag) {
            const long long t0 = clock64();
            while (clock64() - t0 < 2000000) {
            }
        }
        tc_fence_after();
        tmem_dealloc(tmem, kTmemCols);
    }
    if (kTrace && threadIdx.x == kSoftmaxThreads) {  // lane 0 of the MMA warp knows the block count
        const int cta = blockIdx.x;
        if (cta < 1024) {
            long long t1;
            unsigned smid;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1));
            asm volatile("mov.u32 %0, %%smid;" : "=r"(smid));
            long long* row = tp.trace + (64 + cta) * 8;
            row[0] = cta_t0;
            row[1] = t1;
            row[2] = smid;
            row[3] = blocks_done;
            row[4] = cta_c0;
            row[5] = clock64();
        }
    }
}

}  // namespace

namespace tc5 {

// ---- host side --------------------------------------------------------------------------

namespace {
using EncodeFn = CUresult (*)(
    CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
    const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
    CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeFn encode_fn() {
    static EncodeFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult res;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &res) == cudaSuccess &&
            res == cudaDriverEntryPointSuccess) {
            fn = reinterpret_cast<EncodeFn>(sym);
        }
    });
    return fn;
}

}  // namespace

int* status_word(int** device_view) {
    // One pinned, device-mapped word per process: kernels record a wait that ran out
    // there and the host reads it without a synchronisation.
    static int* host = nullptr;
    static int* dev = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        if (cudaHostAlloc(reinterpret_cast<void**>(&host), sizeof(int), cudaHostAllocMapped) == cudaSuccess) {
            *host = 0;
            if (cudaHostGetDevicePointer(reinterpret_cast<void**>(&dev), host, 0) != cudaSuccess) dev = nullptr;
        }
    });
    if (device_view) *device_view = dev;
    return host;
}

long long* g_trace = nullptr;  // set by ktt_b200_set_trace; read at every launch

namespace {
// Encoded maps by what they were encoded from: a decode loop or a training step presents the
// same (pointer, shape, strides) call after call, and a map is a pure function of them.
struct MapKey {
    const void* base;
    int64_t rows, heads, batch, strides[3];
    int d, box_rows, slot[3];
    bool operator==(const MapKey& o) const { return std::memcmp(this, &o, sizeof(MapKey)) == 0; }
};
struct MapEntry {
    MapKey key;
    CUtensorMap map;
    bool used;
};
constexpr int kMapSlots = 256;   // direct-mapped
MapEntry g_maps[kMapSlots];
std::mutex g_maps_lock;

size_t map_slot(const MapKey& k) {
    uint64_t h = 1469598103934665603ull;
    const unsigned char* bytes = reinterpret_cast<const unsigned char*>(&k);
    for (size_t i = 0; i < sizeof(MapKey); ++i) h = (h ^ bytes[i]) * 1099511628211ull;
    return static_cast<size_t>(h % kMapSlots);
}
}  // namespace

bool encode_map(
    CUtensorMap* map, const void* base, int d, int64_t rows, int64_t heads, int64_t batch,
    const int64_t strides[3], const DimOrder& order, int box_rows, const char** why) {
    EncodeFn fn = encode_fn();
    if (!fn) {
        *why = "cuTensorMapEncodeTiled is not available";
        return false;
    }
    MapKey key;
    std::memset(&key, 0, sizeof(key));   // padding bytes take part in the comparison
    key.base = base;
    key.rows = rows;
    key.heads = heads;
    key.batch = batch;
    key.d = d;
    key.box_rows = box_rows;
    for (int i = 0; i < 3; ++i) {
        key.strides[i] = strides[i];
        key.slot[i] = order.slot_of[i];
    }
    const size_t at = map_slot(key);
    {
        std::lock_guard<std::mutex> hold(g_maps_lock);
        if (g_maps[at].used && g_maps[at].key == key) {
            *map = g_maps[at].map;
            return true;
        }
    }
    cuuint64_t dims[4] = {static_cast<cuuint64_t>(d), 1, 1, 1};
    cuuint64_t str[4] = {0, 0, 0, 0};  // str[i] = byte stride of dim i + 1
    cuuint32_t box[4] = {64, 1, 1, 1};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    const int64_t sizes[3] = {rows, heads, batch};
    for (int i = 0; i < 3; ++i) {
        const int slot = order.slot_of[i];
        dims[slot] = static_cast<cuuint64_t>(sizes[i]);
        str[slot - 1] = static_cast<cuuint64_t>(strides[i]) * 2;
        if (i == 0) box[slot] = static_cast<cuuint32_t>(box_rows);
    }
    const CUresult rc = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, str, box, estr,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                           CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (rc != CUDA_SUCCESS) {
        *why = "cuTensorMapEncodeTiled refused the tensor layout";
        return false;
    }
    {
        std::lock_guard<std::mutex> hold(g_maps_lock);
        g_maps[at].key = key;
        g_maps[at].map = *map;
        g_maps[at].used = true;
    }
    return true;
}

// Effective (row, head, batch) sizes and strides of one operand, with size-1 dims given a
// stride that keeps the ascending order valid; false when the layout cannot be a tensor map.
bool operand_layout(
    const void* base, int64_t rows, int64_t heads, int64_t batch, const int64_t in[3],
    int64_t out[3], const char** why) {
    if (reinterpret_cast<uintptr_t>(base) & 15) {
        *why = "operands must be 16-byte aligned";
        return false;
    }
    // in: (batch, head, row) element strides -> out: (row, head, batch)
    out[0] = in[2];
    out[1] = in[1];
    out[2] = in[0];
    const int64_t sizes[3] = {rows, heads, batch};
    int64_t span = 64;  // a stride for size-1 dims: past everything else
    for (int i = 0; i < 3; ++i) {
        if (sizes[i] > 1) {
            if (out[i] <= 0 || out[i] % 8) {
                *why = "row, head and batch strides must be positive multiples of 8 elements";
                return false;
            }
            span = span > out[i] * sizes[i] ? span : out[i] * sizes[i];
        }
    }
    span = (span + 7) / 8 * 8;
    for (int i = 0; i < 3; ++i) {
        if (sizes[i] <= 1) out[i] = span;
    }
    return true;
}

DimOrder order_of(const int64_t strides[3]) {
    int idx[3] = {0, 1, 2};
    for (int a = 0; a < 3; ++a) {
        for (int c = a + 1; c < 3; ++c) {
            if (strides[idx[c]] < strides[idx[a]]) {
                const int t = idx[a];
                idx[a] = idx[c];
                idx[c] = t;
            }
        }
    }
    DimOrder o;
    for (int pos = 0; pos < 3; ++pos) o.slot_of[idx[pos]] = pos + 1;
    return o;
}

long long* trace_buffer() { return g_trace; }
void set_trace(long long* p) { g_trace = p; }

}  // namespace tc5

bool forward_tc5_takes(const AttnParams& p, const char** why) {
    if (p.d != p.dv || (p.d != 64 && p.d != 128)) {
        *why = "head dim must be 64 or 128 with D == Dv";
        return false;
    }
    if (p.mask_dtype != KTT_B200_MASK_NONE && (p.ms[2] != 0 || p.causal)) {
        // A mask that is one row per (batch, head) (key padding) is applied in the kernel.
        *why = "masks that differ between query rows run on the warp-MMA kernel";
        return false;
    }
    for (int i = 0; i < 3; ++i) {
        if (p.os[i] % 8) {
            *why = "output strides must be multiples of 8 elements";
            return false;
        }
    }
    if (reinterpret_cast<uintptr_t>(p.out) & 15) {
        *why = "the output must be 16-byte aligned";
        return false;
    }
    const int64_t tq = p.cu_q ? p.total_q : p.sq, tk = p.cu_q ? p.total_k : p.sk;
    const int64_t bq = p.cu_q ? 1 : p.batch;
    int64_t s[3];
    return operand_layout(p.q, tq, p.heads, bq, p.qs, s, why) &&
           operand_layout(p.k, tk, p.kv_heads, bq, p.ks, s, why) &&
           operand_layout(p.v, tk, p.kv_heads, bq, p.vs, s, why);
}

template <int D>
int launch_tc5(const AttnParams& p, cudaStream_t stream) {
    using P = Plan<D>;
    constexpr int BN = kBN;
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
    if (!encode_map(&mq, p.q, D, tq, p.heads, bq, sq, orders[0], kBM, &why) ||
        !encode_map(&mk, p.k, D, tk, p.kv_heads, bq, sk, orders[1], BN, &why) ||
        !encode_map(&mv, p.v, D, tk, p.kv_heads, bq, sv, orders[2], BN, &why)) {
        return fail(KTT_B200_ERR_UNSUPPORTED, "tcgen05 forward: %s", why);
    }
    Tc5Params tp;
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
    for (int o = 0; o < 3; ++o) {
        for (int i = 0; i < 3; ++i) tp.dim_of[o][i] = orders[o].slot_of[i];
    }
    constexpr int smem = P::kBytes;
    const bool masked = p.mask_dtype != KTT_B200_MASK_NONE;
    auto kernel = masked ? (tp.trace ? fwd_tc5_kernel<D, true, true> : fwd_tc5_kernel<D, false, true>)
                         : (tp.trace ? fwd_tc5_kernel<D, true, false> : fwd_tc5_kernel<D, false, false>);
    if (int rc = ensure_smem(kernel, smem, "cudaFuncSetAttribute(fwd_tc5)")) return rc;
    tp.q_tiles = (p.sq + kBM - 1) / kBM;
    tp.by_heads = divisor_of(p.heads);
    tp.by_batch = divisor_of(p.batch > 0 ? p.batch : 1);
    tp.by_kv_heads = divisor_of(p.kv_heads);
    tp.by_group = divisor_of(p.heads / p.kv_heads);
    tp.by_per_pair = divisor_of(tp.q_tiles > 0 ? tp.q_tiles * (p.heads / p.kv_heads) : 1);
    const int64_t work = static_cast<int64_t>(p.heads) * p.batch * tp.q_tiles;
    if (work > 0x7fffffff) return fail(KTT_B200_ERR_UNSUPPORTED, "tcgen05 forward: too many query tiles");
    tp.work = static_cast<int>(work);
    // K / V that fit L2 comfortably (126 MB on B200) are read from HBM once whatever the
    // order, and the fixed deal of the length-sorted list is then the faster one (measured:
    // 940 against 857 TFLOP/s on 67 MB of K / V). Larger problems take the grouped order,
    // which needs the counter. A caller that passes just a counter (4..255 bytes) asks for
    // drawn work either way (kernels that share the GPU with communication kernels).
    const int64_t kv_rows = p.cu_q ? p.total_k : static_cast<int64_t>(p.batch) * p.sk;
    const int64_t kv_bytes = kv_rows * p.kv_heads * (p.d + p.dv) * 2;
    const bool large = kv_bytes > (96ll << 20);
    const bool explicit_counter = p.fwd_work_counter && !p.fwd_done_counter;
    tp.work_counter = (large || explicit_counter) ? p.fwd_work_counter : nullptr;
    tp.done_counter = tp.work_counter ? p.fwd_done_counter : nullptr;
    tp.grouped = (tp.work_counter && large) ? 1 : 0;
    int dev = 0, sms = 148;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const int grid = tp.work < sms ? tp.work : sms;  // persistent: one CTA per SM
    kernel<<<grid, P::kThreads, smem, stream>>>(mq, mk, mv, tp);
    return check_cuda(cudaGetLastError(), "fwd_tc5 launch");
}

void set_trace_buffer(long long* device_buffer) { tc5::set_trace(device_buffer); }
long long* get_trace_buffer() { return tc5::trace_buffer(); }

int launch_forward_tc5(const AttnParams& p, cudaStream_t stream) {
    if (p.d == 64) return launch_tc5<64>(p, stream);
    return launch_tc5<128>(p, stream);
}

namespace {
// One warp waits, with a short limit, on a barrier nobody arrives at: the wait gives up,
// records its code in the status word and the kernel returns normally.
__global__ void wait_timeout_kernel(int* status, long long limit) {
    __shared__ uint64_t barrier;
    __shared__ int abort_flag;
    if (threadIdx.x == 0) {
        mbar_init(smem_u32(&barrier), 1);
        abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncwarp();
    const bool got = mbar_wait_slow(smem_u32(&barrier), 0, &abort_flag, 999, status, limit);
    if (got && threadIdx.x == 0) atomicCAS_system(status, 0, 998);   // cannot happen: nobody arrives
}
}  // namespace

int selftest_wait_timeout(cudaStream_t stream) {
    int* dev_status = nullptr;
    if (!status_word(&dev_status) || !dev_status) return fail(KTT_B200_ERR_LAUNCH, "no status word");
    wait_timeout_kernel<<<1, 32, 0, stream>>>(dev_status, 100000);
    return check_cuda(cudaGetLastError(), "wait_timeout launch");
}

int device_status(int* code) {
    int* host = status_word(nullptr);
    if (!host || *host == 0) {
        if (code) *code = 0;
        return 0;
    }
    if (code) *code = *host;
    *host = 0;
    note_call(5);
    return KTT_B200_ERR_DEVICE_WAIT;
}

}  // namespace ktt
