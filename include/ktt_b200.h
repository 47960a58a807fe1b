/* C ABI of the B200 flash-attention library (libktt_b200.so).
 *
 * Torch-free: every tensor crosses as a raw device pointer plus element strides, every
 * scalar as a plain C type. The caller owns and allocates all memory (outputs, softmax
 * statistics, gradients, workspaces); the library only launches kernels on the stream
 * it is given. Convention follows the reference's C ABI
 * (src/kohakutt_native/csrc/py_bridge/ktt_capi.h:1-16): a call returns 0 on success
 * and a negative status on failure, with the message in a thread-local buffer read by
 * ktt_b200_last_error(); nothing throws across the boundary.
 *
 * All tensors are bf16 unless noted; the innermost (head-dim) stride must be 1.
 */
#pragma once
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define KTT_B200_API __attribute__((visibility("default")))
#define KTT_B200_ABI_VERSION 1

/* Status codes (all failures are negative). */
enum {
    KTT_B200_OK = 0,
    KTT_B200_ERR_UNSUPPORTED = -1, /* shape / dtype / layout the kernels do not take */
    KTT_B200_ERR_BAD_ARGUMENT = -2, /* null pointer, negative size, bad lengths */
    KTT_B200_ERR_LAUNCH = -3,       /* a CUDA call or kernel launch failed */
    KTT_B200_ERR_DEVICE_WAIT = -4,  /* a bounded in-kernel wait ran out */
};

/* Mask element types of ktt_b200_attn_args.mask_dtype. */
enum {
    KTT_B200_MASK_NONE = 0,
    KTT_B200_MASK_BOOL = 1, /* uint8, nonzero keeps the key */
    KTT_B200_MASK_BF16 = 2, /* additive */
    KTT_B200_MASK_F32 = 3,  /* additive */
    KTT_B200_MASK_F16 = 4,  /* additive */
};

/* Causal alignment. Dense calls are top-left (query i sees keys <= i,
 * aten_attention.cpp:431-436); packed calls are bottom-right (query r of a sequence
 * sees its first min(Lk, r + 1 + Lk - Lq) keys, ktt_flash/varlen_plan.hpp:40-42,70). */
enum {
    KTT_B200_CAUSAL_NONE = 0,
    KTT_B200_CAUSAL_TOP_LEFT = 1,
    KTT_B200_CAUSAL_BOTTOM_RIGHT = 2,
};

/* Kernel choice of ktt_b200_attn_args.kernel. */
enum {
    KTT_B200_KERNEL_AUTO = 0,
    KTT_B200_KERNEL_MMA = 1,  /* general warp-MMA kernels: any head dim <= 256, masks */
    KTT_B200_KERNEL_TC5 = 2,  /* TMA + tcgen05/TMEM kernels: head dim 64 / 128 */
    KTT_B200_KERNEL_TC5_WIDE = 3,  /* forward only: the head-dim-128 tcgen05 kernel's design also at
                                      head dim 64, where KERNEL_TC5 picks the two-stream kernel */
};

/* One attention problem, dense ([B, H, S, D] with arbitrary batch/head/row strides, so
 * head views of [B, S, H*D] storages are read in place) or packed ([T, H, D] with
 * cu_seqlens). Strides are in elements, ordered (batch, head, row); packed calls pass
 * batch stride 0 and rows are offset by cu_seqlens[b].
 *
 * Replaces the operand list of bridge::sdpa / sdpa_train / sdpa_varlen / sdpa_lengths
 * (src/kohakutt_native/csrc/core/device/tt_bridge.hpp:925-1095). */
typedef struct ktt_b200_attn_args {
    int32_t batch;     /* B, or the number of packed sequences */
    int32_t heads;     /* H query heads */
    int32_t kv_heads;  /* Hk, divides H */
    int32_t sq;        /* query rows per batch; packed: the longest sequence (max_q) */
    int32_t sk;        /* key rows per batch; packed: max_k */
    int64_t total_q;   /* packed: rows of q (Tq); dense: ignored */
    int64_t total_k;   /* packed: rows of k and v (Tk); dense: ignored */
    int32_t d;         /* head dim of q and k */
    int32_t dv;        /* head dim of v and out */
    int32_t causal;    /* KTT_B200_CAUSAL_* */
    float scale;       /* softmax scale (multiplies q.k) */
    int32_t kernel;    /* KTT_B200_KERNEL_* */

    const void* q;
    const void* k;
    const void* v;
    void* out;         /* bf16, caller-allocated */
    float* lse;        /* natural-log row log-sum-exp, fp32; may be NULL on forward */
    int64_t q_strides[3];
    int64_t k_strides[3];
    int64_t v_strides[3];
    int64_t out_strides[3];
    int64_t lse_strides[3]; /* dense [B,H,Sq]: (H*Sq, Sq, 1); packed [H,Tq]: (0, Tq, 1) */

    /* Optional mask broadcastable to [B, H, Sq, Sk]; stride 0 broadcasts a dim. For a
     * packed call the key index is the packed key index (mask [Tk], strides 0,0,0,1).
     * Additive values are clamped below at -5e5; a bool mask turns a dropped key's
     * logit into -5e5 (ktt_flash/varlen_plan.hpp:12-17, program.cpp:912-919). */
    const void* mask;
    int32_t mask_dtype; /* KTT_B200_MASK_* */
    int64_t mask_strides[4];

    /* Optional per-batch key counts, int32 [B] on the device, clamped to [1, sk] by
     * the kernel (ktt_flash/reader.cpp:111-160); never read on the host. */
    const int32_t* key_lengths;

    /* Packed calls: int32 [batch + 1] on the device; NULL for dense calls. */
    const int32_t* cu_seqlens_q;
    const int32_t* cu_seqlens_k;

    /* Backward only (NULL on forward). dk / dv are already summed over each GQA group. */
    const void* dout;
    void* dq;
    void* dk;
    void* dv_out;
    int64_t dout_strides[3];
    int64_t dq_strides[3];
    int64_t dk_strides[3];
    int64_t dv_strides[3];
    /* Backward: workspace of ktt_b200_sdpa_backward_workspace() bytes, 256-byte aligned.
     * Forward (optional): ktt_b200_sdpa_forward_workspace() bytes, 16-byte aligned,
     * zero-filled once before the first use. With it the CTAs draw their query tiles from a
     * counter there instead of a fixed deal, and the head-dim-128 kernel orders the tiles so
     * that those in flight share the K / V of a few (batch, head) pairs (problems whose K / V
     * exceed L2 otherwise re-read them several times). The kernel leaves the counter zero;
     * calls that share a buffer must not overlap on the GPU. The head-dim-128 kernel also
     * takes 4 to 255 bytes: one int32 the caller zero-fills before EVERY call. */
    void* workspace;
    int64_t workspace_bytes;
} ktt_b200_attn_args;

/* Decode: one (or a few) query tokens per sequence against a static KV cache, split over
 * the sequence. q [B, H, Sq<=16/group, D], cache k / v [B, Hk, Smax, D / Dv].
 * Replaces ktt::_sdpa_lengths on the decode route (aten_lengths.cpp:69-99,
 * aten_attention.cpp:578-604). */
typedef struct ktt_b200_decode_args {
    int32_t batch, heads, kv_heads;
    int32_t sq;        /* query tokens per sequence; heads/kv_heads * sq <= 16 */
    int32_t sk;        /* cache capacity Smax */
    int32_t d, dv;     /* 64 or 128, equal */
    float scale;
    const void* q;
    const void* k;
    const void* v;
    void* out;
    float* lse;        /* optional [B, H, Sq] */
    int64_t q_strides[3];
    int64_t k_strides[3];
    int64_t v_strides[3];
    int64_t out_strides[3];
    const int32_t* key_lengths; /* int32 [B] on the device, or NULL for sk everywhere */
    int32_t splits;    /* 0 = choose; else the number of sequence splits */
    void* scratch;     /* ktt_b200_decode_scratch_bytes() bytes, 256-byte aligned, zero-filled
                          once before its first use (the kernel leaves its counters zero) */
    int64_t scratch_bytes;
} ktt_b200_decode_args;

/* ktt_abi_version (ktt_capi.h:13). */
KTT_B200_API int ktt_b200_abi_version(void);
/* ktt_last_error (ktt_capi.h:14): message of this thread's last failing call. */
KTT_B200_API const char* ktt_b200_last_error(void);

/* ktt_counters (ktt_capi.h:24-26) reduced to this path: out[8] = forward calls on the
 * tcgen05 kernel, forward calls on the warp-MMA kernel, backward calls, decode calls,
 * refused calls, device-wait timeouts, backward calls on the tcgen05 kernels, reserved. */
KTT_B200_API int ktt_b200_counters(int64_t* out8);
KTT_B200_API int ktt_b200_reset_counters(void);

/* Device-side failure report, the counterpart of the reference stream's "first failing op
 * is raised at the next call" (csrc/core/device/stream.hpp:11-47). Every wait inside the
 * tcgen05 kernels is bounded; one that runs out records a code in a host-visible word.
 * Returns 0, or KTT_B200_ERR_DEVICE_WAIT with *code set (and clears the word). Call it
 * after synchronising the stream; the next forward call also checks it. */
KTT_B200_API int ktt_b200_device_status(int* code);

/* Test support for the report above: launches one warp that waits, with a limit of ~1e5
 * cycles, on a barrier nobody arrives at. The wait gives up (code 999), the kernel returns
 * normally and the device stays healthy; after a synchronize ktt_b200_device_status reports
 * KTT_B200_ERR_DEVICE_WAIT, as does the next tcgen05 launch. Nothing faults, traps or spins
 * for longer than the limit. */
KTT_B200_API int ktt_b200_selftest_wait_timeout(void* stream);

/* Measurement support: reads `bytes` (a multiple of 16, 16-byte aligned) of device memory
 * once with 16-byte loads dealt grid-stride over two CTAs per SM, and discards them. What a
 * plain read of a buffer of that size reaches on this GPU is the yardstick the decode
 * kernel's GB/s is put beside; `sink` (one int32) only keeps the loads alive. No
 * counterpart in the reference. */
KTT_B200_API int ktt_b200_probe_read(const void* data, int64_t bytes, int32_t* sink, void* stream);

/* Debug dump of one query tile, the counterpart of the reference's FLASH_DUMP build
 * (ktt_flash/program.hpp:56-65, aten_attention.cpp:814-831: `_debug_flash_dump(q, k, v,
 * is_causal, row)`, the intermediate tiles of one query tile row). While a device buffer is
 * set, every head-dim-64 tcgen05 forward launch runs its traced instantiation, and the
 * tile (batch, head, q_tile: rows q_tile * 128 ..) writes out what its row threads hold,
 * straight from their registers:
 *   per key block j < max_blocks, KTT_B200_DUMP_BLOCK_FLOATS floats:
 *     x [128][128]   the exponents, logit * scale * log2(e) (+ mask term) - reference, -inf
 *                    where the key is hidden;
 *     p [128][128]   2^x as the bf16 values that feed P V;
 *     m [2][128]     the reference maximum of each half row (keys 0-63, 64-127 of the block)
 *                    while this block was processed (it moves only when a block exceeds it
 *                    by 2^8, and the two halves of a row agree on it);
 *   then, at float offset max_blocks * KTT_B200_DUMP_BLOCK_FLOATS:
 *     o [128][64]    the unnormalised output accumulator at the end of the tile (of a tile
 *                    shared by a CTA's two streams: after their halves were merged);
 *     m [128], l [128]   the final reference maximum and the row sum; lse = ln 2 (m + log2 l).
 * Blocks of a shared tile's second half are measured against that stream's own reference.
 * Entries of rows or blocks the tile does not have are left as they were. Null clears the
 * request. Process-wide, like the trace buffer; not meant for concurrent launches. */
#define KTT_B200_DUMP_BLOCK_FLOATS (2 * 128 * 128 + 2 * 128)
#define KTT_B200_DUMP_TAIL_FLOATS (128 * 64 + 2 * 128)
KTT_B200_API int ktt_b200_set_dump(float* device_buffer, int32_t batch, int32_t head, int32_t q_tile, int32_t max_blocks);

/* Profiling zones, the counterpart of the reference's FLASH_PROFILE device zones
 * (ktt_flash/compute.cpp:25-30, program.hpp:56-65): with a device buffer of 64 x 8 int64
 * set, CTA (0, 0, 0) of every tcgen05 forward launch stamps clock64 per key block (slots:
 * S ready, pass 1 done, previous P V done, pass 2 done, P published, MMA lane before the
 * next Q K^T, after the wait for P, after issuing P V), and rows 64 .. 64 + 1023 receive per
 * CTA its start and end on the global nanosecond timer, its SM and its key-block count; the
 * buffer then holds (64 + 1024) x 8 int64. (The head-dim-64 forward's slots per key block:
 * S ready, maximum known, exponentials done, P published, first chunk loaded, its
 * exponentials done, previous P V done, second chunk loaded; row 60 holds its epilogue:
 * last P V done, outputs written, row sums exchanged and, for a tile the CTA's two streams
 * share, the other stream's half published, read, merged.)
 * The decode kernel writes, per CTA, rows 64.. with six nanosecond stamps: start,
 * dependency wait over, lengths scanned, first tile landed, stream done, end. The tcgen05
 * backward writes, per CTA, rows 64..: start, end, SM, CTA index, set-up done, first scores,
 * last MMA done, results stored; and for the first 56 CTAs, per score warp, rows
 * 64 + 512 + 8 CTA + warp: the clocks its item loop spent meeting, waiting for S, in phase 1,
 * waiting for dP, in phase 2, and the item count. kohaku_tt_b200/trace.py reads all three.
 * NULL turns it off (default). */
KTT_B200_API int ktt_b200_set_trace(void* device_buffer);

/* ktt_flash::supports / refusal (ktt_flash/program.cpp:847-910): 1 when the forward
 * kernels take the problem, 0 with the reason in ktt_b200_last_error(). Launches
 * nothing and touches no device memory. */
KTT_B200_API int ktt_b200_sdpa_supported(const ktt_b200_attn_args* args);
/* ktt_flash::supports_backward (ktt_flash/program.cpp:1529-1585). */
KTT_B200_API int ktt_b200_sdpa_backward_supported(const ktt_b200_attn_args* args);

/* Forward of dense or packed attention: ktt_sdpa / ktt_sdpa_train (ktt_capi.h:122-125),
 * bridge::sdpa_varlen and bridge::sdpa_lengths (tt_bridge.hpp:925-1095). Writes out and,
 * when args->lse is set, the natural-log row statistics. */
KTT_B200_API int ktt_b200_sdpa_forward(const ktt_b200_attn_args* args, void* stream);

/* Bytes of the optional forward workspace for the problem (0 when the kernel that will run
 * uses none). No counterpart in the reference: its host planner deals the chunks to cores
 * before the launch (ktt_flash/program.cpp:204-242,269-275); here the deal happens on the
 * device. */
KTT_B200_API int64_t ktt_b200_sdpa_forward_workspace(const ktt_b200_attn_args* args);
/* Query tiles the head-dim-64 forward kernel keeps in flight per SM of the current device
 * (2: one CTA with two streams; 0 means a build or device the kernel was not sized for).
 * Launches nothing. */
KTT_B200_API int ktt_b200_forward_streams_per_sm(void);

/* Bytes of workspace ktt_b200_sdpa_backward needs for the problem (0 on error). */
KTT_B200_API int64_t ktt_b200_sdpa_backward_workspace(const ktt_b200_attn_args* args);
/* Backward (dq, dk, dv with the softmax recomputed from lse): ktt_sdpa_train_backward
 * (ktt_capi.h:126-135), bridge::sdpa_varlen_backward, bridge::sdpa_lengths_backward. */
KTT_B200_API int ktt_b200_sdpa_backward(const ktt_b200_attn_args* args, void* stream);

/* Split-K decode against a static KV cache. */
KTT_B200_API int64_t ktt_b200_decode_scratch_bytes(const ktt_b200_decode_args* args);
KTT_B200_API int ktt_b200_decode(const ktt_b200_decode_args* args, void* stream);

/* ktt_b200_decode for callers that must not allocate device memory while they run (a
 * server that hands out all of the GPU at start-up and gives a plugin only input and
 * output buffers; a decode loop that cannot afford the device-wide stall a cudaMalloc can
 * cause). It has no counterpart in the reference. The split-K partials go to a fixed
 * 4 MiB array inside the library, so args->scratch and args->scratch_bytes are ignored
 * and the call makes no allocation of any kind.
 *  - A call whose partials exceed 4 MiB (more than 207 (batch, kv head) pairs at head dim
 *    128 on a 148-SM GPU, 696 at head dim 64) is refused with KTT_B200_ERR_UNSUPPORTED.
 *  - The first call on a device does a one-time set-up (address of the array, kernel
 *    attributes); make it before any stream capture.
 *  - Every call on a device uses the same array. It needs no clearing between calls, but
 *    calls that overlap on the GPU (different streams, no ordering) corrupt each other:
 *    keep them on one stream or order them with events.
 *  - The array is the current device's: call with the device current whose stream is passed.
 *  - Every GPU that loads the library holds the 4 MiB until the process ends. */
KTT_B200_API int ktt_b200_decode_static(const ktt_b200_decode_args* args, void* stream);

/* One decode step with its neighbours fused in: the rotate-half rotary embedding of the
 * new query and key (ktt.rotary: csrc/aten/nn/aten_fused.cpp:30-43, bridge::rotary,
 * device_attention.cpp:1340-1356), the write of the new key / value row into the static
 * cache (the `index_copy_` that is 20 % of a decode token in the reference's profile,
 * docs/reference/results.md:296) and attention over the old keys plus the new one.
 *
 * base: as for ktt_b200_decode with sq == 1; base.q is the query BEFORE rotary; base.k /
 * base.v are the caches and are written: row lengths[b] of each (b, kv head) receives the
 * rotated key / the value. base.key_lengths[b] is the number of keys already cached,
 * clamped to [0, sk - 1]; attention sees lengths[b] + 1 keys. The lengths themselves are
 * not changed; lengths_out, when set (a different buffer), receives lengths[b] + 1.
 * k_new [B, Hk, D], v_new [B, Hk, D] bf16 with (batch, head) element strides, rows dense.
 * cos / sin: bf16 rows of D values, rope_row_stride elements apart; row lengths[b] when
 * rope_by_position is non-zero (a [positions, D] table), else row b (one row per batch).
 * y = x * cos + cat(-x[D/2:], x[:D/2]) * sin, products and sum rounded separately in fp32,
 * result rounded to bf16 before it is used or stored. */
typedef struct ktt_b200_decode_append_args {
    ktt_b200_decode_args base;
    const void* k_new;
    const void* v_new;
    int64_t k_new_strides[2];
    int64_t v_new_strides[2];
    const void* cos;
    const void* sin;
    int64_t rope_row_stride;
    int32_t rope_by_position;
    int32_t* lengths_out; /* optional int32 [B] */
} ktt_b200_decode_append_args;

KTT_B200_API int ktt_b200_decode_append(const ktt_b200_decode_append_args* args, void* stream);

/* Merge of two partial attention results over disjoint key sets (ring attention steps):
 * out / lse [rows] are updated in place with (out2, lse2). fp32 lse; out_is_f32 = 0: out and
 * out2 bf16, 1: both fp32, 2: fp32 out (an accumulator) with bf16 out2 (a kernel's output).
 * rows = B*H*S rows of dv values, row stride dv. No reference counterpart: the reference
 * has no sequence-parallel attention. */
KTT_B200_API int ktt_b200_merge_partials(
    void* out, float* lse, const void* out2, const float* lse2,
    int64_t rows, int32_t dv, int32_t out_is_f32, void* stream);

#ifdef __cplusplus
}
#endif
