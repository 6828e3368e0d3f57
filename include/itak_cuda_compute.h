/*
 * itak_cuda_compute.h - C ABI of the B200 (sm_100a) KV-cache hot path.
 *
 * This is the boundary a `crates/cuda-compute` backend crate binds over FFI to
 * implement the engine's `Compute::attention` step with backend-owned KV, the
 * speculation seam (checkpoint / rewind / release) and the prefix-KV seam
 * (snapshot capture / install).  Plain pointers and sizes only; no C++ or
 * torch types cross it.  Each entry point names the reference interface it
 * stands in for (paths relative to the reference repository root).
 *
 * Conventions
 *  - Every call returns an itk_status.  0 is success; every refusal is a named
 *    code mirroring one variant of the reference's error enums, and the text of
 *    the last refusal is available from itk_last_error().  A refused call
 *    leaves the backend's state exactly as it was (validate, then mutate).
 *  - A backend owns `n_slots` resident sequences ("slots").  Calls on one
 *    backend are serialised by the caller (the reference backend is not Sync).
 *  - Rows arrive already RoPE'd: RoPE is the caller's job, as in
 *    crates/attention/src/attention.rs:5-8 - except through the *_prep calls,
 *    which normalise and rotate raw rows on the device first.
 *  - "host" pointers may be pageable or pinned; "device" pointers must be
 *    device memory on the backend's device, 16-byte aligned.
 *  - There is no CPU fallback: every data-path call launches CUDA kernels and
 *    fails with ITK_ERR_CUDA when no device is usable.
 */
#ifndef ITAK_CUDA_COMPUTE_H
#define ITAK_CUDA_COMPUTE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Refusal codes.  1..14 mirror crates/attention/src/error.rs:9-127
 * (AttentionError), 32..46 mirror crates/itak-kv/src/error.rs (KvError),
 * 64 is the backend's own StepFailed{step, detail}
 * (crates/cpu-compute/src/cpu.rs:28-33).  100+ have no counterpart: they are
 * limits of a device-resident cache with a fixed allocation. */
typedef enum itk_status {
    ITK_OK = 0,
    ITK_ERR_ZERO_DIMENSION = 1,
    ITK_ERR_INVALID_WINDOW = 2,
    ITK_ERR_SIZE_OVERFLOW = 3,
    ITK_ERR_SHAPE_MISMATCH = 4,
    ITK_ERR_INVALID_LAYER = 5,
    ITK_ERR_OUT_OF_ORDER_POSITION = 6,
    ITK_ERR_NON_DIVISIBLE_HEADS = 7,
    ITK_ERR_NO_VISIBLE_KEYS = 8,
    ITK_ERR_CHECKPOINT_BUSY = 9,
    ITK_ERR_STALE_CHECKPOINT = 10,
    ITK_ERR_CHECKPOINT_TOO_DEEP = 11,
    ITK_ERR_CHECKPOINT_RANGE_EXCEEDED = 12,
    ITK_ERR_BULK_RESTORE_NOT_FRESH = 13,
    ITK_ERR_REWIND_OUT_OF_RANGE = 14,
    ITK_ERR_INCOHERENT_CACHE = 32,
    ITK_ERR_INCONSISTENT_SNAPSHOT = 33,
    ITK_ERR_BAD_MAGIC = 34,
    ITK_ERR_UNSUPPORTED_VERSION = 35,
    ITK_ERR_TRUNCATED = 36,
    ITK_ERR_CHECKSUM_MISMATCH = 37,
    ITK_ERR_GEOMETRY_MISMATCH = 38,
    ITK_ERR_FINGERPRINT_MISMATCH = 39,
    ITK_ERR_EMPTY_PREFIX = 40,
    ITK_ERR_TOKEN_COUNT_MISMATCH = 41,
    ITK_ERR_PREFIX_HASH_MISMATCH = 42,
    ITK_ERR_SNAPSHOT_TOKEN_MISMATCH = 43,
    ITK_ERR_ENTRY_TOO_LARGE = 44,
    ITK_ERR_INVALID_CONFIG = 45,
    ITK_ERR_IO = 46,
    ITK_ERR_STEP_FAILED = 64,
    ITK_ERR_CUDA = 100,
    ITK_ERR_INVALID_ARGUMENT = 101,
    ITK_ERR_CAPACITY = 102,
    ITK_ERR_INVALID_SLOT = 103
} itk_status;

typedef enum itk_kv_dtype {
    ITK_KV_F32 = 0, /* the reference CPU cache's format (crates/attention/src/cache.rs:11-15) */
    ITK_KV_F16 = 1  /* IEEE half, round-to-nearest-even on append, NaN -> sign|0x7e00
                       (crates/wgpu-compute/src/kernels/k1_q4k_gemv.rs:285-329) */
} itk_kv_dtype;

/* Shape of one backend.  Stands in for the (GlimmerConfig -> CacheShape)
 * binding of crates/cpu-compute/src/cpu.rs:171-244 plus the session limits of
 * crates/wgpu-compute/src/session.rs:235-249. */
typedef struct itk_config {
    uint32_t n_layers;
    const uint32_t* layer_window; /* per layer: 0 = global, w > 0 = sliding window of w; NULL = all global */
    uint32_t q_heads;
    uint32_t kv_heads;
    uint32_t head_dim;
    uint32_t n_slots;     /* resident sequences */
    uint32_t max_context; /* positions a slot can hold on a global layer */
    uint32_t chunk_cap;   /* most rows one attention call may carry per sequence; a windowed
                             layer's ring holds window + chunk_cap positions */
    int32_t kv_dtype;     /* itk_kv_dtype */
    int32_t device;       /* CUDA device ordinal */
} itk_config;

typedef struct itk_backend itk_backend;   /* opaque */
typedef struct itk_snapshot itk_snapshot; /* opaque, device-resident prefix snapshot */

/* Receipt of a live checkpoint: crates/attention/src/cache.rs:229-273.
 * `id` names the slot's cache instance, so a handle presented to another
 * sequence (or after a reset) is stale by construction. */
typedef struct itk_checkpoint {
    uint64_t id;
    uint64_t serial;
    uint64_t base; /* position of every layer when the checkpoint was taken */
    uint64_t max_round_tokens;
} itk_checkpoint;

/* Per-call counters (SessionStats, crates/wgpu-compute/src/session.rs:493-540). */
typedef struct itk_stats {
    uint64_t attention_calls;
    uint64_t kernel_launches;
    uint64_t rows_appended;
    uint64_t kv_bytes_read; /* algorithmic: visible keys x Hkv x D x 2 x element size */
    uint64_t prefix_captures;
    uint64_t prefix_restores;
    uint64_t last_splits; /* KV splits chosen by the last decode launch */
} itk_stats;

/* ---- lifetime ------------------------------------------------------------ */

/* KvCache::new for every slot (crates/attention/src/cache.rs:327-371): same
 * refusal order (empty layer list, zero kv heads, zero head dim, zero window,
 * size overflow), then q_heads % kv_heads, then the device allocation. */
int itk_backend_create(const itk_config* cfg, itk_backend** out);
void itk_backend_destroy(itk_backend* b);
/* Text of the last refusal on `b`; with b == NULL, of the last failed create. */
const char* itk_last_error(const itk_backend* b);
/* Work is issued on `cuda_stream` (a cudaStream_t) from now on; NULL selects
 * the backend's own non-blocking stream again (pass cudaStreamLegacy for
 * CUDA's default stream).  The caller orders its own work against it. */
int itk_set_stream(itk_backend* b, void* cuda_stream);
/* Tuning and A/B switches of one backend, set explicitly by the caller (the library reads no environment
 * variables); no counterpart in the reference, whose switches live in the engine's configuration
 * (crates/itak-kv/src/config.rs).  Names: "decode_ctas" (persistent CTAs of the decode kernel, 0 = two per SM),
 * "decode_splits" (KV splits of the general and multi-row kernels, 0 = chosen per launch), "pdl" (programmatic
 * dependent launch inside the replayable loop, default 1), "decode_fused_sum" (cells shared by many CTAs are summed
 * in L2, default 1), "separate_append" (the append kernel runs as a launch of its own instead of the attention
 * kernel storing the call's new rows, default 0), "force_general" (multi-row calls on an f16 cache and every call
 * on an f32 cache take the CUDA-core kernel, default 0), "verify_tc" (multi-row calls take the
 * tcgen05 kernel, default 1), "gather_poll_limit" (polls of a peer's arrival flag before the fused gather's wait
 * gives up, default 200000), "decode_lanes" (two-lane schedule of the gathering loop: 0 never, 1 when a launch is
 * short enough to gain, 2 whenever possible; default 1), "decode_lane_stagger" (how far the second lane of a step's
 * first launch starts behind the first, in per cent of the time the first needs to stream its keys; default 100),
 * "layers_host_bulk_bytes" (itk_attention_layers_host: a forward that uploads no more than this many bytes sends
 * all layers' rows up in three copies, launches the layers back to back and brings the results down in one copy,
 * instead of pipelining per-layer copies against the kernels; default 1 MiB (where a layer's kernel is shorter than its copies' fixed cost), 0 = always pipeline).
 * "layers_host_decode_loop" (itk_attention_layers_host: a decode step - one row per sequence on an f16 cache - that
 * uploads no more than this many bytes runs as one step of the replayable loop behind three strided uploads;
 * default 8 MiB, 0 = never),
 * "tc_wait_kclocks" (bound of every wait inside the tcgen05 multi-row kernel, in units of 1024 SM clocks; 0 = the
 * default of about a second) and "tc_withhold_first_tile" (for tests of that kernel's give-up path only: the first
 * key tile of every CTA is loaded but never reported, so the wait for it runs out, every role leaves its loop, the
 * launch's outputs are not valid and the next synchronising call returns ITK_ERR_CUDA; default 0).
 * Unknown names and out-of-range values are refused; not allowed inside
 * a resident loop. */
int itk_set_option(itk_backend* b, const char* name, int64_t value);
int itk_synchronize(itk_backend* b);
int itk_get_stats(const itk_backend* b, itk_stats* out);
/* Per-kernel device timing, the counterpart of the reference's timestamp-query
 * diagnostics (crates/wgpu-compute/src/timestamps.rs:1-140).  While enabled,
 * every attention and append kernel launch is bracketed by a CUDA event pair on
 * the launching stream (up to `capacity` pairs, created up front).
 * itk_profile_read synchronises the stream and returns the summed kernel
 * milliseconds and launch counts since the last enable; capacity 0 disables. */
int itk_profile_enable(itk_backend* b, uint32_t capacity);
int itk_profile_read(itk_backend* b, double* attention_ms, uint64_t* attention_launches, double* append_ms,
                     uint64_t* append_launches);
/* The snapshot gather / restore scatter launches summed by the last itk_profile_read. */
int itk_profile_read_copy(itk_backend* b, double* copy_ms, uint64_t* copy_launches);

/* ---- the attention step ---------------------------------------------------- */

/* Compute::attention for one sequence (crates/muse-glimmer/src/compute.rs:29-42,82;
 * crates/cpu-compute/src/cpu.rs:506-655).  Host buffers: q [rows][q_heads*D],
 * k and v [rows][kv_heads*D], out [rows][q_heads*D].  `position` is the
 * caller's Cache::position(); a backend whose layer is elsewhere refuses with
 * ITK_ERR_STEP_FAILED naming both positions (cpu.rs:565-581).  Appends the
 * rows at position.., then attends each row causally (and within the window on
 * sliding layers).  Returns after the result is in `out`. */
int itk_attention(itk_backend* b, uint32_t slot, uint32_t layer, const float* q, size_t q_len, const float* k,
                  size_t k_len, const float* v, size_t v_len, uint64_t position, float* out);

/* The same step for `n_seqs` slots at once, `rows` rows each (continuous
 * batching; the reference runs one OS thread and one backend per slot,
 * crates/itak-engine/src/engine.rs:4-15).  q [n_seqs][rows][q_heads*D],
 * k, v [n_seqs][rows][kv_heads*D], out like q.  Host buffers. */
int itk_attention_batch(itk_backend* b, uint32_t layer, uint32_t n_seqs, const uint32_t* slots,
                        const uint64_t* positions, uint32_t rows, const float* q, const float* k, const float* v,
                        float* out);

/* The attention step of EVERY layer of one forward in one call, for a caller that holds all layers' projections
 * on the host (a benchmark of the path alone, a replay of recorded activations): host q [layers][n_seqs][rows][q_heads*D],
 * k, v [layers][n_seqs][rows][kv_heads*D], out like q; every slot must sit at positions[i] on every layer.  The
 * backend pipelines the layers over three streams - layer l's rows upload while layer l-1 computes and layer l-2's
 * result downloads - and returns after the last result is in `out`; a decode step on an f16 cache that moves little
 * (option "layers_host_decode_loop") runs as one step of the replayable loop (itk_resident_begin / layer / end) behind three strided uploads; another small forward (option
 * "layers_host_bulk_bytes") sends every layer's rows up in three strided copies, launches the layers back to
 * back and brings all results down in one copy, since per-layer copies would cost more than their overlap hides.  Same refusals as itk_attention_batch, all
 * layers validated before anything is queued.  The first call allocates the per-layer staging.  No counterpart in
 * the reference, whose forward calls Compute::attention layer by layer (crates/muse-glimmer/src/model.rs:452-462). */
int itk_attention_layers_host(itk_backend* b, uint32_t n_seqs, const uint32_t* slots, const uint64_t* positions,
                              uint32_t rows, const float* q, const float* k, const float* v, float* out);

/* As itk_attention_batch with q, k, v, out resident in device memory; returns
 * once the work is queued on the backend's stream. */
int itk_attention_batch_device(itk_backend* b, uint32_t layer, uint32_t n_seqs, const uint32_t* slots,
                               const uint64_t* positions, uint32_t rows, const float* d_q, const float* d_k,
                               const float* d_v, float* d_out);

/* Attention preparation on the device: per-head RMSNorm of the Q and K rows and their rotary rotation, done by
 * the backend ahead of the append, so that the projections' raw rows never leave the device to be rotated.
 * Stands in for the reference's fused preparation K9 (crates/wgpu-compute/src/kernels/k9_attn_prep.rs:74-236)
 * and for the rotation inside the CPU backend's attention step (crates/cpu-compute/src/cpu.rs:598-622, which
 * rotates on sliding-window layers only).  The arithmetic is the CPU reference's: f64 mean of squares and f64
 * angles, each result rounded once to f32 (crates/torch-math/src/norm.rs:21-53, rope_interleaved.rs:65-117,
 * rope.rs:63-117); results agree with it to the last bit or two of f32, not bit for bit.
 * A NULL weight skips that norm; rotary_dim 0 skips the rotation.  Weights are host pointers, copied. */
typedef struct itk_prep_config {
    const float* q_norm_weight; /* [head_dim] or NULL */
    const float* k_norm_weight; /* [head_dim] or NULL */
    float norm_eps;             /* finite, > 0 when a weight is given */
    float rope_base;            /* finite, > 1 when rotary_dim != 0 */
    uint32_t rotary_dim;        /* 0, or even and <= head_dim */
    uint32_t pairing;           /* 0 = adjacent pairs (2i, 2i+1) as rope_interleaved; 1 = half split (i, i + rotary_dim/2) as rope */
} itk_prep_config;
int itk_layer_prep_set(itk_backend* b, uint32_t layer, const itk_prep_config* cfg);
/* itk_attention_batch / itk_attention_batch_device taking the projections' raw Q and K rows: prepares them as the
 * layer's configuration says, then appends and attends as those calls do.  Same shapes, same refusals. */
int itk_attention_batch_prep(itk_backend* b, uint32_t layer, uint32_t n_seqs, const uint32_t* slots,
                             const uint64_t* positions, uint32_t rows, const float* q, const float* k, const float* v,
                             float* out);
int itk_attention_batch_prep_device(itk_backend* b, uint32_t layer, uint32_t n_seqs, const uint32_t* slots,
                                    const uint64_t* positions, uint32_t rows, const float* d_q, const float* d_k,
                                    const float* d_v, float* d_out);

/* A decode loop whose launches depend on no host-side position, so that one step can be recorded once (a
 * CUDA graph) and replayed - the counterpart of the reference session's "one command buffer per forward"
 * (crates/wgpu-compute/src/session.rs:3230-3233).  The listed slots must sit at one position on every layer,
 * with an f16 cache and head_dim 64 or 128.
 *   itk_resident_begin    reserves `max_steps` decode steps for the slots and writes their positions to the device
 *   itk_resident_layer    one layer of the current step for all listed slots: stores the new K/V row and attends
 *                         (device f32 q/out [n_seqs][q_heads*D], k/v [n_seqs][kv_heads*D]); only queues work
 *   itk_resident_advance  queues the kernel that moves every listed slot to the next position (end of a step)
 *   itk_resident_end      tells the backend how many steps actually ran, and leaves the mode
 * Between begin and end no other call may touch the listed slots. */
/* How the replayable loop's decode launch cuts its work: for `n_seqs` sequences of keys[] visible keys, each with
 * `cells_per_seq` (KV head x head chunk) cells of ceil(keys / 64) tiles, across `ctas` persistent CTAs with `splits`
 * partial slots per cell.  *aligned = 1 when every cell gets a whole number of CTAs of its own (no CTA crosses a cell
 * boundary), 0 for equal contiguous runs over all cells laid end to end.  runs[cta] = {sequence, cell within the
 * sequence, first tile, tiles walked (0 = idle), CTAs sharing the first cell, this CTA's number among them}; a run
 * that ends a cell goes on with the next cell's first tile.  Host arithmetic only - the same functions the kernel
 * evaluates - so that the partition can be checked without a GPU.  No counterpart in the reference, whose kernels
 * take one workgroup per (row, head) (crates/wgpu-compute/src/kernels/k6_attention.rs:286-296). */
int itk_decode_plan(const uint32_t* keys, uint32_t n_seqs, uint32_t cells_per_seq, uint32_t ctas, uint32_t splits,
                    uint32_t* aligned, uint32_t* runs);
/* How an ordinary decode call (one row per sequence, f16 cache) cuts a batch into launches: at most
 * *seqs_per_launch sequences go into one launch, whose (sequence, KV head x head chunk) cells then own
 * *parts_per_cell partial slots each of the backend's split scratch of *scratch_slots slots (a cell can always be
 * cut in two, so never fewer than 2).  ITK_ERR_CAPACITY when a single sequence's cells do not fit.  Host arithmetic
 * only, the function the backend itself uses; no counterpart in the reference. */
int itk_decode_batch_limits(uint32_t n_seqs, uint32_t cells_per_seq, uint32_t* seqs_per_launch, uint32_t* parts_per_cell,
                            uint64_t* scratch_slots);
int itk_resident_begin(itk_backend* b, uint32_t n_seqs, const uint32_t* slots, uint64_t max_steps);
int itk_resident_layer(itk_backend* b, uint32_t layer, const float* d_q, const float* d_k, const float* d_v,
                       float* d_out);
int itk_resident_advance(itk_backend* b);
int itk_resident_end(itk_backend* b, uint64_t steps_done);

/* The per-layer gather of head outputs across the GPUs of one box, done by the decode kernel itself (no
 * counterpart in the reference, which is single-GPU).  Every rank owns a KV-head shard (a backend created with
 * its share of the heads).  Each rank creates one gather buffer, the ranks exchange the 64-byte handles (any
 * host channel) and open each other's; inside the replayable loop itk_resident_layer_gather then behaves like
 * itk_resident_layer, except that the CTA finishing a (sequence, head) cell stores its rows - plain stores to
 * peer-mapped memory over NVLink - at `gather_offset_bytes` of EVERY rank's buffer (the caller gives each rank
 * and layer its own offset), and counts the cell on every rank's arrival counters, kept per sequence of the loop
 * and source rank in the buffer's header.  A short launch runs as two lanes - the batch cut in two halves of about
 * equal work, half of the grid's CTAs each - which the backend keeps out of phase, so that one half's outputs cross
 * NVLink while the other half streams its cache (a layer's inputs for a sequence depend on the previous layer's
 * gathered outputs of that sequence only).  Before a CTA of the loop uses its inputs it checks, with a bounded wait,
 * that all ranks' cells of the previous launch have arrived for the sequences it works on
 * (itk_gather_status reports a wait that ran out: bit 0 of *error_bits; the kernel then carries on, its own outputs
 * do not depend on the peers' rows).  All ranks must call itk_gather_reset, then synchronise with
 * each other, before itk_resident_begin; a step of the loop must launch every layer exactly once. */
int itk_gather_create(itk_backend* b, uint32_t world, uint32_t rank, uint64_t data_bytes, void** local_data,
                      uint8_t* handle64);
int itk_gather_open(itk_backend* b, uint32_t peer_rank, const uint8_t* handle64);
/* As itk_gather_open for a peer whose buffer this process can already address - another backend of the same
 * process (one process driving several GPUs with peer access enabled), or memory mapped by the caller's own
 * symmetric-memory allocator: `peer_local_data` is the pointer itk_gather_create returned as *local_data on that
 * peer.  The mapping stays the caller's. */
int itk_gather_attach(itk_backend* b, uint32_t peer_rank, void* peer_local_data);
/* Unmaps every peer's buffer (this rank's own stays until the backend is destroyed).  For an orderly shutdown every
 * rank calls this, the ranks synchronise, and only then the backends are destroyed - so that no rank frees a buffer
 * a peer still maps. */
int itk_gather_close_peers(itk_backend* b);
int itk_gather_reset(itk_backend* b);
int itk_gather_status(itk_backend* b, uint32_t* error_bits);
int itk_resident_layer_gather(itk_backend* b, uint32_t layer, const float* d_q, const float* d_k, const float* d_v,
                              uint64_t gather_offset_bytes);

/* Draft-model (DFlash) attention, the attention half of the reference's K17
 * (crates/wgpu-compute/src/kernels/k17_dflash.rs:109-251; CPU form crates/dflash/src/model.rs:388-466): `rows`
 * query rows at positions block_start.. attend a position-addressed, possibly sparse set of `committed` rows (row
 * of position p at p * kv_heads * key_len in d_committed_k, p * kv_heads * value_len in d_committed_v; the list
 * d_committed_positions says which exist) together with the block's own `block_rows` K/V rows, non-causally unless
 * `causal`, and within `window` when `sliding` (key kp is hidden from query qp when kp <= qp - window, signed).
 * All pointers are device f32 / u32; q [rows][q_heads][key_len], out [rows][q_heads][value_len].  No backend handle:
 * the draft's cache is the caller's (crates/dflash/src/cache.rs:1-24).  key_len and value_len up to 256.  Only queues
 * work on `cuda_stream`; refusals (the names of k17_dflash.rs:276-316) come back as ITK_ERR_INVALID_ARGUMENT with the
 * text in error_text. */
int itk_draft_attention(const float* d_q, const float* d_committed_k, const float* d_committed_v,
                        const uint32_t* d_committed_positions, uint32_t committed, const float* d_block_k,
                        const float* d_block_v, uint32_t block_start, uint32_t rows, uint32_t block_rows,
                        uint32_t q_heads, uint32_t kv_heads, uint32_t key_len, uint32_t value_len, uint32_t causal,
                        uint32_t sliding, uint32_t window, float scale, float* d_out, void* cuda_stream,
                        char* error_text, size_t error_text_len);

/* The rotate half of the reference's K17 (crates/wgpu-compute/src/kernels/k17_dflash.rs:78-107, 255-271): rotates
 * `rows` x `heads` head rows of d_x ([rows][heads][head_dim], device f32) in place, row r at d_positions[r] (device
 * u32) - positions need not be consecutive, as an injection chunk's are not.  pairing 1 is the draft model's
 * half-split (NeoX) form, torch_math::rope (crates/torch-math/src/rope.rs:63-117); pairing 0 is rope_interleaved.  f64
 * angles rounded once, as the CPU functions.  Only queues work on `cuda_stream`; refusals come back as
 * ITK_ERR_INVALID_ARGUMENT with the text in error_text. */
int itk_rope_rows(float* d_x, const uint32_t* d_positions, uint32_t rows, uint32_t heads, uint32_t head_dim,
                  uint32_t rotary_dim, uint32_t pairing, float base, void* cuda_stream, char* error_text,
                  size_t error_text_len);

/* gqa_attention alone (crates/attention/src/attention.rs:104-215) over what a
 * slot already holds: `rows` queries at query_positions[], host buffers.
 * Refuses ITK_ERR_NO_VISIBLE_KEYS when a query sees nothing. */
int itk_gqa_attention(itk_backend* b, uint32_t slot, uint32_t layer, const float* q, size_t q_len, uint32_t rows,
                      const uint64_t* query_positions, float* out);

/* ---- KvCache-level operations ------------------------------------------------ */

/* KvCache::append (crates/attention/src/cache.rs:423-474): one position's K
 * and V rows, host f32.  Same check order: k length, v length, live
 * checkpoint range, layer, position == appended. */
int itk_append(itk_backend* b, uint32_t slot, uint32_t layer, const float* k, size_t k_len, const float* v,
               size_t v_len, uint64_t position);
/* `rows` consecutive positions start.. in one call, host f32 [rows][kv_heads*D]. */
int itk_append_rows(itk_backend* b, uint32_t slot, uint32_t layer, const float* k, const float* v, uint32_t rows,
                    uint64_t start);
/* The same append for `n_seqs` slots with device-resident f32 sources
 * [n_seqs][rows][kv_heads*D] (prefill of a resident cache without a host round
 * trip); slot i receives rows at starts[i]..  Queued on the backend's stream. */
int itk_append_rows_device(itk_backend* b, uint32_t layer, uint32_t n_seqs, const uint32_t* slots,
                           const uint64_t* starts, uint32_t rows, const float* d_k, const float* d_v);
/* KvCache::next_position / stored_len (cache.rs:407-415). */
int itk_next_position(const itk_backend* b, uint32_t slot, uint32_t layer, uint64_t* out);
int itk_stored_len(const itk_backend* b, uint32_t slot, uint32_t layer, uint64_t* out);
/* The gather behind KvCache::view (cache.rs:581-585, 836-904): the visible rows
 * of one layer, oldest first, [rows][kv_heads][D] in the cache's element type
 * (2 or 4 bytes each), copied to host buffers holding at least
 * stored_len * kv_heads * D elements.  keys or values may be NULL. */
int itk_view_gather(itk_backend* b, uint32_t slot, uint32_t layer, void* keys, void* values,
                    uint64_t* first_position, uint64_t* rows);
/* KvCache::restore_bulk (cache.rs:513-577): install rows for positions
 * first_position.. on a fresh layer, host f32 [rows][kv_heads*D]. */
int itk_restore_bulk(itk_backend* b, uint32_t slot, uint32_t layer, uint64_t first_position, const float* keys,
                     size_t keys_len, const float* values, size_t values_len);
/* CpuCompute::reset (crates/cpu-compute/src/cpu.rs:264-267) for one slot:
 * drops the sequence, its checkpoint and its cache identity. */
int itk_reset(itk_backend* b, uint32_t slot);

/* ---- speculation seam ---------------------------------------------------------- */

/* CpuCompute::cache_checkpoint / KvCache::checkpoint (cpu.rs:281-295,
 * cache.rs:634-717).  On the device ring (window + chunk_cap rows, one more
 * than the reference session's ring of crates/wgpu-compute/src/session.rs:235-249)
 * a round of at most chunk_cap rows never overwrites a row that a later query
 * or a later view can reach, so nothing is copied; a bound above chunk_cap on
 * a model with sliding layers refuses with ITK_ERR_CHECKPOINT_TOO_DEEP. */
int itk_cache_checkpoint(itk_backend* b, uint32_t slot, uint64_t max_round_tokens, itk_checkpoint* out);
/* CpuCompute::cache_rewind / KvCache::rewind_to (cpu.rs:309-322, cache.rs:758-818):
 * truncate every layer of the slot to `target` positions, target in
 * [base, appended].  The checkpoint stays live. */
int itk_cache_rewind(itk_backend* b, uint32_t slot, const itk_checkpoint* cp, uint64_t target);
/* CpuCompute::cache_release / KvCache::release (cpu.rs:326-339, cache.rs:824-833). */
int itk_cache_release(itk_backend* b, uint32_t slot, const itk_checkpoint* cp);

/* ---- prefix-KV seam --------------------------------------------------------------- */

/* ResidentSession::capture_prefix_snapshot / KvSnapshot::capture
 * (crates/wgpu-compute/src/session.rs:4827-4887, crates/itak-kv/src/snapshot.rs:247-302):
 * every layer's visible rows in absolute-position order, kept in device memory
 * in the cache's element type.  Refuses layers at different positions. */
int itk_snapshot_capture(itk_backend* b, uint32_t slot, itk_snapshot** out);
/* ResidentSession::install_prefix_snapshot / KvSnapshot::restore
 * (session.rs:4925-4971, snapshot.rs:321-334): validate the whole snapshot
 * against the backend's geometry, then reset the slot and scatter the rows to
 * their slots; the slot ends at position token_count. */
int itk_snapshot_restore(itk_backend* b, uint32_t slot, const itk_snapshot* snap);
void itk_snapshot_free(itk_snapshot* snap);
uint64_t itk_snapshot_token_count(const itk_snapshot* snap);
uint64_t itk_snapshot_payload_bytes(const itk_snapshot* snap);
/* One layer block copied to host in the cache's element type,
 * [rows][kv_heads][D]; either pointer may be NULL. */
int itk_snapshot_layer_to_host(itk_backend* b, const itk_snapshot* snap, uint32_t layer, void* keys, void* values,
                               uint64_t* first_position, uint64_t* rows);
/* Build a device snapshot from host f32 rows in the layout of the ITKV format's
 * layer blocks (crates/itak-kv/src/snapshot.rs:13-29): for each layer,
 * first_position[l], rows[l], keys[l] and values[l] as [rows][kv_heads*D].
 * Values are converted to the cache's element type as an append would. */
int itk_snapshot_from_host_f32(itk_backend* b, uint64_t token_count, const uint64_t* first_position,
                               const uint64_t* rows, const float* const* keys, const float* const* values,
                               itk_snapshot** out);

/* KvSnapshot::to_bytes (crates/itak-kv/src/snapshot.rs:13-29, 381-415): the versioned `ITKV` byte format -
 * magic, version 1, model fingerprint, token count, KV heads, head dim, per-layer headers (kind, window, first
 * position, row count), per-layer keys then values as little-endian f32, FNV-1a-64 checksum.  An f16 cache is
 * written as the exact f32 values of its elements, so the bytes are an ordinary version-1 snapshot.  Two-call
 * protocol: with out == NULL only *size is set. */
int itk_snapshot_to_itkv(itk_backend* b, const itk_snapshot* snap, const char* model_fingerprint, uint8_t* out,
                         size_t capacity, size_t* size);
/* The same with the format version chosen.  Version 1 is the reference's (f32 rows, what itk_snapshot_to_itkv
 * writes).  Version 2 is this library's extension for f16 caches, which the reference refuses to snapshot
 * (crates/wgpu-compute/src/session.rs:383-398): one more header field - a u32 element type directly after the
 * version, 0 = f32, 1 = IEEE half - and the rows stored in that type, so an f16 cache's prefix takes half the bytes
 * and its bit patterns survive a round trip untouched.  itk_snapshot_from_itkv reads both (half rows bound for an
 * f32 cache are widened exactly; f32 rows bound for an f16 cache are rounded as an append rounds). */
int itk_snapshot_to_itkv_version(itk_backend* b, const itk_snapshot* snap, const char* model_fingerprint,
                                 uint32_t version, uint8_t* out, size_t capacity, size_t* size);
/* KvSnapshot::from_bytes followed by restore_checked's trust checks (snapshot.rs:425-540, 345-371): strict
 * decode (bad magic, unknown version or element type, truncation, layer count beyond the buffer, overflowing
 * products, trailing bytes, checksum, self-consistency - each a named refusal), then the backend's geometry and, when
 * expected_fingerprint is not NULL, the model fingerprint.  Rows are cast to the cache's element type. */
int itk_snapshot_from_itkv(itk_backend* b, const uint8_t* bytes, size_t n, const char* expected_fingerprint,
                           itk_snapshot** out);

/* The strict decode alone (KvSnapshot::from_bytes + validate, crates/itak-kv/src/snapshot.rs:187-236, 425-540), host
 * code only: vets ITKV bytes of either format version without a backend or a device.  Returns ITK_OK and the
 * header's version, token count and bytes per stored element, or the refusal's code with its text in `why`. */
int itk_itkv_check(const uint8_t* bytes, size_t n, uint32_t* version, uint64_t* token_count, uint32_t* elem_bytes,
                   char* why, size_t why_len);

/* ---- for callers that cannot allocate ------------------------------------------------ */

/* No counterpart in the reference (its backends allocate freely).  Decode
 * attention - one query row per sequence over an f16 cache in this library's
 * head-major layout - for a caller that is not allowed to allocate device
 * memory when it calls: a server that sized everything at start-up, a plugin
 * living inside another runtime's allocator, a latency-critical loop that
 * cannot afford cudaMalloc's synchronisation, or work being recorded for
 * replay.  The split-K partials live in a fixed ~8.1 MiB array inside the
 * library image (present on every GPU that loads the library, until exit), so
 * the call performs no cudaMalloc / cudaFree and needs no backend object.
 *
 *   k_layer, v_layer  device, f16 [slot][kv_heads][ring][head_dim]; keys 0..kv_len[i]-1 of sequence i
 *                     sit at rows 0.. of slot slots[i]
 *   d_q, d_out        device f32 [n_seqs][q_heads][head_dim]
 *   splits            CTAs along each key range, at most 64; 0 picks one
 *   error_text        optional buffer that receives the reason of a refusal
 *
 * Limits: head_dim 64 or 128; n_seqs <= 64; n_seqs x kv_heads x ceil(group/8) x max(splits, 2) <= 2048
 * (a key range can always be cut in two, so one split still reserves two partial slots).
 * Larger requests return ITK_ERR_CAPACITY.  k_layer, v_layer, d_q and d_out must be 16-byte aligned.
 * The first call on a device looks up the array's device address and sets a kernel attribute (under a
 * lock, so first calls from several host threads are safe); issue that first
 * call outside any stream capture.  All calls share the array (the counters in
 * it are cleared on the stream at the start of each call): calls that may
 * overlap on the GPU must be serialised by the caller.  The device that owns
 * the buffers must be current.  Returns once the work is queued on the stream. */
int itk_decode_attention_noalloc(const void* k_layer, const void* v_layer, uint32_t ring, uint32_t kv_heads,
                                 uint32_t q_heads, uint32_t head_dim, uint32_t n_seqs, const uint32_t* slots,
                                 const uint32_t* kv_len, const float* d_q, float* d_out, uint32_t splits,
                                 void* cuda_stream, char* error_text, size_t error_text_len);

/* ---- the persistent prefix store ------------------------------------------------ */

/* PrefixStore (crates/itak-kv/src/store.rs): one file per entry under `root`, keyed by token prefix, bounded by
 * `max_bytes` with least-recently-used eviction; same entry bytes and file names as the reference's store (layout
 * store.rs:5-21), so a directory can be shared with it.  Host code only.  An entry's payload is a snapshot in the
 * ITKV encoding (itk_snapshot_to_itkv / itk_snapshot_from_itkv).  Calls on one store are serialised by the caller.
 *   open     store.rs:147-170: refuses a zero cap (ITK_ERR_INVALID_CONFIG), creates the root, indexes every
 *            well-formed "*.kv" entry; malformed files are left on disk, unindexed, and named by
 *            itk_prefix_store_last_refusal.  itk_prefix_store_last_error(NULL) has the text of a failed open.
 *   put      store.rs:236-303: refuses an empty prefix, a snapshot whose token count differs from the id count, an
 *            entry larger than the cap; writes a temp file, syncs, renames; then evicts least recently used entries
 *            (never the new one) until the store is within its cap.  `now` is the caller's clock (unix seconds).
 *   lookup   store.rs:314-452: the longest stored prefix of `query` that passes every trust check - ids hash back
 *            to the key, ids equal the query's prefix, payload decodes whole and covers the preamble's token count,
 *            and, when given, the required geometry (n_layers, layer_window, kv_heads, head_dim of an itk_config)
 *            and fingerprint match.  A candidate that fails is refused by name and the search goes on to shorter
 *            prefixes.  A hit restamps the entry's last-used time in place.  *token_count == 0 is a clean miss;
 *            the returned bytes belong to the store until its next call. */
typedef struct itk_prefix_store itk_prefix_store;
int itk_prefix_store_open(const char* root, uint64_t max_bytes, itk_prefix_store** out);
void itk_prefix_store_close(itk_prefix_store* s);
const char* itk_prefix_store_last_error(const itk_prefix_store* s);
const char* itk_prefix_store_last_refusal(const itk_prefix_store* s);
int itk_prefix_store_rescan(itk_prefix_store* s);
int itk_prefix_store_put(itk_prefix_store* s, const uint32_t* tokens, size_t n_tokens, const uint8_t* itkv, size_t itkv_len,
                         uint64_t now);
int itk_prefix_store_lookup(itk_prefix_store* s, const uint32_t* query, size_t n_query, const itk_config* required_geometry,
                            const char* required_fingerprint, uint64_t now, uint64_t* token_count, const uint8_t** itkv,
                            size_t* itkv_len);
int itk_prefix_store_stats(const itk_prefix_store* s, uint64_t* entries, uint64_t* total_bytes, uint64_t* max_bytes);
/* Entry `i` of the index, longest prefix first (store.rs:179-184). */
int itk_prefix_store_entry(const itk_prefix_store* s, uint64_t i, char* file_name, size_t file_name_cap, uint64_t* prefix_hash,
                           uint64_t* token_count, uint64_t* bytes, uint64_t* created_unix, uint64_t* last_used_unix);

#ifdef __cplusplus
}
#endif
#endif /* ITAK_CUDA_COMPUTE_H */
