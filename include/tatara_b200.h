/*
 * tatara_b200 -- C ABI of the B200 (sm_100a) attention + Gated DeltaNet operators.
 *
 * This header is the drop-in boundary for the reference engine's attention hot path.
 * The reference talks to its GPU through (pipeline name, buffer-slot bindings, u32
 * constants, grid) tuples; every entry point below replaces one such dispatch and cites
 * the reference call site whose slot order it keeps.  Conventions shared by all calls:
 *
 *   - Plain C, int status return, caller-owned DEVICE pointers, explicit CUDA stream
 *     (passed as void* == cudaStream_t; NULL is the default stream).
 *   - Nothing is allocated after tatara_ctx_create ("the per-token walk allocates
 *     nothing", include/tatara/runtime/decode_step.h:110-114).
 *   - bf16 storage / f32 arithmetic.  Tensor layouts are the reference's:
 *       attention projection  [row][9216] = per head h: q(256)|gate(256), k(2x256), v(2x256)
 *       q / gate / attended   [row][16][256] bf16
 *       KV cache planes K, V  [kv_head][capacity][256] bf16   (attention.metal:108-111)
 *       partial record        258 f32 = [numerator(256) | max | sum]  (decode_geometry.h:111)
 *       GDN projection        [row][12352] = q 2048|k 2048|v 4096|z 4096|b 32|a 32
 *       GDN conv state        [3][8192] bf16 oldest first; conv weights [8192][4] bf16
 *       GDN recurrent state   [32 v-head][128 v-dim][128 k-dim] f32 (in/out ping-pong)
 *   - Arguments are validated on the host BEFORE anything is enqueued
 *     (src/runtime/decode_step.cpp:812-824); a failing call enqueues nothing.
 *   - Calls are asynchronous on `stream`; errors of earlier asynchronous work surface
 *     as TATARA_CUDA_ERROR from a later call or from tatara_ctx_sync.
 *   - The block kernels that use thread-block clusters and tensor memory (tatara_attn_prefill,
 *     tatara_project_dense) are issued with nothing else of this library in flight on the
 *     device: keep them in the stream that carries the rest of the work.  Issued beside other
 *     streams' kernels they have stalled (cause not established); the host layer's owner loop
 *     (tatara_b200/host/wave_loop.hpp) therefore uses one stream.
 */
#ifndef TATARA_B200_H_
#define TATARA_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Status codes; names mirror MetalCommandError
 * (include/tatara/backend/metal/commands.h:232-262). */
typedef enum tatara_status {
    TATARA_OK = 0,
    TATARA_INVALID_BUFFER = 1,          /* null / misaligned pointer            */
    TATARA_CONTEXT_OUT_OF_RANGE = 2,    /* context >= capacity, empty key range */
    TATARA_STATE_SLOT_MISMATCH = 3,     /* aliasing in/out state slots          */
    TATARA_INVALID_STREAM_GROUP = 4,    /* lane count 0 or above the maximum    */
    TATARA_INVALID_DISPATCH_EXTENT = 5, /* rows == 0, bad chunk size, ...       */
    TATARA_INVALID_DEVICE = 6,
    TATARA_SCRATCH_TOO_SMALL = 7,
    TATARA_DEVICE_WAIT_TIMEOUT = 8,     /* a bounded device-side wait gave up   */
    TATARA_CUDA_ERROR = 9
} tatara_status;

typedef struct tatara_ctx tatara_ctx;

#define TATARA_MAX_LANES 256u            /* lanes per batched call            */
#define TATARA_MAX_CONTEXT 262144u       /* prefill_geometry.h:14             */
#define TATARA_RECORD_FLOATS 258u        /* decode_geometry.h:111             */

/* One row of the per-layer lane table (the reference's state_table rows,
 * src/runtime/decode_step.cpp:1037-1062).  Offsets are in ELEMENTS of the pool's type. */
typedef struct tatara_attn_lane {
    uint64_t kv_offset; /* element offset of this lane's stripe in the K and V pools */
    uint32_t context;   /* position of the token being decoded; attends 0..context    */
    uint32_t reserved;
} tatara_attn_lane;

typedef struct tatara_gdn_lane {
    uint64_t conv_in, conv_out; /* element offsets into the conv pool (bf16)      */
    uint64_t rec_in, rec_out;   /* element offsets into the recurrent pool (f32)  */
} tatara_gdn_lane;

/* ---- context ----------------------------------------------------------------------- */
/* Replaces device/queue/library/pipeline creation (tools/native/decode_harness.cpp:148-337). */
tatara_status tatara_ctx_create(int device, tatara_ctx** out);
void tatara_ctx_destroy(tatara_ctx* ctx);
/* Waits for `stream` and returns the first latched device-side error, if any
 * (MetalExecutionResult, include/tatara/backend/metal/commands.h:374-387). */
tatara_status tatara_ctx_sync(tatara_ctx* ctx, void* stream);
const char* tatara_last_error_string(const tatara_ctx* ctx);
const char* tatara_status_name(tatara_status status);
int tatara_abi_version(void);
/* Kernels launched through this context since creation (for benchmark accounting). */
uint64_t tatara_ctx_launch_count(const tatara_ctx* ctx);

/* Execution policy of a context: choices that change how a kernel runs and never what it computes
 * (the reference keeps such choices in policy structs fixed at boot: DecodeAttentionSplitPolicy,
 * include/tatara/runtime/decode_step.h:15-21; PrefillExecutionPolicy, prefill_step.h:42-73).
 * Set before the first call that the policy affects, not between calls in flight. */
typedef enum tatara_policy {
    /* Cap on the rows of K and of V of each decode CTA's partition that are requested into L2 before
     * the kernel waits for its predecessor in the stream (the kernel asks for a quarter of the
     * partition up to this cap; 0 switches the requests off). */
    TATARA_POLICY_DECODE_L2_PREFETCH_KEYS = 0,
    /* Which implementation evaluates tatara_gdn_prefill with chunk 64: 0 = the tensor-memory form
     * (tcgen05 MMAs fed by TMA, the state as an f32 accumulator in tensor memory) as ONE launch in which
     * the scan of early chunks runs beside the preparation of later ones, 2 = the same kernels as two
     * launches, 1 = the register-resident mma.sync form.  Same algebra, same tolerance against the
     * sequential scan. */
    TATARA_POLICY_GDN_CHUNK_FORM = 1,
    /* Which kernel evaluates tatara_attn_prefill: 0 = CTA pairs (two SMs on the same 128 query rows of two
     * heads of a KV group, each loading half of every K and V tile), 1 = one CTA per (query tile, head).
     * Same arithmetic in the same order: the outputs are bit-identical. */
    TATARA_POLICY_ATTN_PREFILL_FORM = 2,
    /* How the fused GDN decode step (tatara_gdn_decode_batch, _indirect) moves the 64 KiB of state each CTA
     * reads and rewrites: 0 = cp.async.bulk copies through shared memory, 1 = per-lane loads into registers and
     * streaming stores.  Same arithmetic: the outputs are bit-identical. */
    TATARA_POLICY_GDN_DECODE_FORM = 3,
    /* Where the records of a single-lane tatara_attn_decode are merged: 0 (default) = in a second kernel that is
     * staged while the partition kernel runs, as the batched and the split calls do; 1 = in the partition kernel's
     * own launch (its CTAs count their finished items and then take the 64 (head, quarter) pieces).  Same
     * arithmetic in the same order: bit-identical.  Measured slower by 0.4 - 2 us at every context (the merge
     * then runs on 4 warps per piece behind two more trips to L2), which is why it is not the default. */
    TATARA_POLICY_DECODE_FUSED_MERGE = 4,
    /* How tatara_q4_project brings the weights of one to four rows in: 0 (default) = whole column groups by
     * cp.async.bulk copies into shared memory, asked for before the dependency wait; 1 = per-lane loads two
     * blocks ahead of the arithmetic.  Same chains and trees: bit-identical. */
    TATARA_POLICY_Q4_ROW_FORM = 5,
    /* 1 = the fused GDN decode step lets the next kernel of its stream be staged while it computes (programmatic
     * dependent launch).  The caller's promise: no kernel that follows within the next few launches reads, before
     * its own dependency wait, the recurrent or conv state this call writes -- true of a layer walk (the out
     * projection follows, then another layer), false of a loop that steps ONE state back to back, because the
     * step asks for its state rows before it waits.  0 (default) = the step's dependents start when it has
     * finished. */
    TATARA_POLICY_GDN_STEP_EARLY_DEPENDENTS = 6
} tatara_policy;
tatara_status tatara_ctx_set_policy(tatara_ctx* ctx, tatara_policy policy, uint64_t value);
uint64_t tatara_ctx_get_policy(const tatara_ctx* ctx, tatara_policy policy);

/* ---- geometry (pure functions; include/tatara/runtime/decode_geometry.h:133-135, 165-273) */
/* Keys per partition and partition count of the split-KV decode for `n_keys` attended
 * keys.  Depends on n_keys only, never on the batch: this is what keeps a lane's output
 * bit-identical alone vs batched (src/runtime/decode_step.cpp:15-19). */
uint32_t tatara_attn_partition_keys(uint32_t n_keys);
uint32_t tatara_attn_partitions(uint32_t n_keys);
/* Scratch bytes that decode of `lanes` lanes, each attending at most `max_keys` keys, needs
 * (attn_record_scratch_bytes, decode_geometry.h:256-262). */
uint64_t tatara_attn_decode_scratch_bytes(uint32_t max_keys, uint32_t lanes);

/* ---- gated full attention ------------------------------------------------------------ */
/* attn_qk_rope / attn_qk_rope_blk: slots 0 projection, 1 q_norm w, 2 k_norm w, 3 q out,
 * 4 gate out, 5 K cache, 6 V cache, 7 context, 8 capacity; grid.y = rows
 * (src/runtime/decode_step.cpp:713-723, src/runtime/prefill_step.cpp:1450-1465).
 * Normalises and rotates q/k for `rows` positions starting at `position` and appends K, V
 * to the cache at those positions. */
tatara_status tatara_attn_qk_rope(tatara_ctx* ctx, void* stream, const void* projection,
                                  const void* q_weight, const void* k_weight, void* q_out,
                                  void* gate_out, void* keys, void* values, uint32_t position,
                                  uint32_t capacity, uint32_t rows);

/* attn_qk_rope_ms: one row per lane over pooled caches; strides in elements
 * (src/backend/metal/kernels/attention.metal:119-198). */
tatara_status tatara_attn_qk_rope_batch(tatara_ctx* ctx, void* stream, const void* projection,
                                        const void* q_weight, const void* k_weight, void* q_out,
                                        void* gate_out, void* keys_pool, void* values_pool,
                                        uint32_t capacity, const tatara_attn_lane* lanes,
                                        uint32_t n_lanes, uint32_t projection_stride,
                                        uint32_t query_stride);

/* Decode attention of one lane: slots 0 q, 1 gate, 2 K, 3 V, 4 context, 5 out, 6 capacity,
 * plus the record scratch of the partitioned family
 * (src/runtime/decode_step.cpp:239-247, 296-337).  Attends keys 0..context inclusive.
 * The decode kernels are programmatic dependent launches: K/V rows below the lane's last
 * partition (rows that cannot be the one a preceding tatara_attn_qk_rope call appends) may be
 * requested while the previous kernel of the stream is still finishing; q, gate, the last
 * partition and every output wait for it.  Library kernels that write more than the appended
 * row keep plain stream order. */
tatara_status tatara_attn_decode(tatara_ctx* ctx, void* stream, const void* q, const void* gate,
                                 const void* keys, const void* values, uint32_t context,
                                 uint32_t capacity, void* out, void* scratch,
                                 uint64_t scratch_bytes);

/* Lane-batched decode: slots 0 q slab, 1 gate slab, 2 K pool, 3 V pool, 4 state_table,
 * 5 out slab, 6 capacity, 8 query_stride (src/runtime/decode_step.cpp:1261-1272).  One
 * varlen launch for every lane; each lane's arithmetic is exactly its solo call's. */
tatara_status tatara_attn_decode_batch(tatara_ctx* ctx, void* stream, const void* q,
                                       const void* gate, const void* keys_pool,
                                       const void* values_pool, const tatara_attn_lane* lanes,
                                       uint32_t n_lanes, uint32_t capacity, uint32_t query_stride,
                                       void* out, void* scratch, uint64_t scratch_bytes);

/* Decode attention of one lane for callers that must not allocate device memory: a serving
 * loop that has frozen its memory plan after boot, a plug-in running inside a host framework
 * whose allocator it may not touch, or any code path where cudaMalloc (a synchronising call
 * that can fail under memory pressure) is off limits.  It has no counterpart in the reference,
 * whose record scratch is always a caller-owned buffer.  Same arithmetic and output as
 * tatara_attn_decode, but the partial records go to a 1.2 MB array built into the library, so
 * no scratch pointer is passed and this call never calls cudaMalloc, cudaFree or any routine
 * that allocates.  Limits and sharing:
 *   - at most 262144 attended keys (context <= 262143, the model's maximum context: a lane is
 *     never cut into more than 74 partitions, which is what the array holds); longer lanes return
 *     TATARA_SCRATCH_TOO_SMALL and must use tatara_attn_decode with caller scratch;
 *   - every call on a device shares the one array: calls that may overlap on the GPU
 *     (different streams, or several host threads) race on it; serialise them.  The array
 *     keeps the previous call's records, which is harmless: each call rewrites every record it
 *     later reads, so nothing has to start at zero;
 *   - the first call on each device (with that device current) looks up the array's device
 *     address and configures the kernel (host threads that make it together are serialised
 *     inside the call); make that first call before any stream capture;
 *   - every GPU that loads the library holds the 1.2 MB until the process exits;
 *   - ctx may be NULL (it only receives the error text and the launch count). */
tatara_status tatara_attn_decode_static(tatara_ctx* ctx, void* stream, const void* q,
                                        const void* gate, const void* keys, const void* values,
                                        uint32_t context, uint32_t capacity, void* out);

/* Split-KV building block: one merged record per head over keys [key_begin, key_end) of a
 * cache slice -> records_out [16][258] f32, un-normalised, no gate
 * (scores/values record family, src/runtime/decode_step.cpp:296-330). */
tatara_status tatara_attn_decode_partial(tatara_ctx* ctx, void* stream, const void* q,
                                         const void* keys, const void* values,
                                         uint32_t key_begin, uint32_t key_end, uint32_t capacity,
                                         void* records_out, void* scratch, uint64_t scratch_bytes);

/* attention_decode_combine: slots records, gate, nparts, out
 * (src/runtime/decode_step.cpp:331-337; attention.metal:1086-1108).
 * Record (head h, part p) sits at records + h*head_stride + p*part_stride (in floats);
 * the reference layout is head_stride = nparts*258, part_stride = 258. */
tatara_status tatara_attn_combine(tatara_ctx* ctx, void* stream, const void* records,
                                  uint32_t nparts, uint64_t head_stride, uint64_t part_stride,
                                  const void* gate, void* out);

/* ---- split-KV of one lane across the GPUs of a box, over peer memory (no counterpart in the
 * reference, which is single-device).  One process per GPU.  Every rank owns a gather buffer
 * [2 parities][world][16][258] f32 and a flag array [2 parities][world] u32 inside one peer
 * buffer that the other ranks map through CUDA IPC. */
/* Allocates (cudaMalloc, zero-filled) a buffer and exports its 64-byte IPC handle; the other
 * ranks open it.  Set-up time only. */
tatara_status tatara_peer_buffer_create(tatara_ctx* ctx, uint64_t bytes, void** ptr, void* handle64);
tatara_status tatara_peer_buffer_open(tatara_ctx* ctx, const void* handle64, void** ptr);
tatara_status tatara_peer_buffer_close(tatara_ctx* ctx, void* ptr, int owned);
/* tatara_attn_decode_partial whose merged record ([16][258]) is stored by the kernel itself into
 * slot `rank` of EVERY rank's gather buffer (peer stores over NVLink), after which word `rank` of
 * every rank's flag array is set to `epoch` (release, system scope).  peer_gather / peer_flags:
 * `world` device pointers (this rank's own buffer at index rank), already offset to the parity
 * in use.  epoch > 0 and different from the previous call's on the same parity. */
tatara_status tatara_attn_decode_partial_push(tatara_ctx* ctx, void* stream, const void* q,
                                              const void* keys, const void* values,
                                              uint32_t key_begin, uint32_t key_end, uint32_t capacity,
                                              void* const* peer_gather, void* const* peer_flags,
                                              uint32_t rank, uint32_t world, uint32_t epoch,
                                              void* scratch, uint64_t scratch_bytes);
/* tatara_attn_combine over this rank's gather buffer ([world][16][258]) that first waits until
 * all `world` flags equal `epoch`.  The wait is bounded by wait_limit_us (<= 2 000 000); when it
 * runs out the kernel writes nothing and tatara_ctx_sync returns TATARA_DEVICE_WAIT_TIMEOUT. */
tatara_status tatara_attn_combine_wait(tatara_ctx* ctx, void* stream, const void* gather,
                                       const void* flags, uint32_t world, uint32_t epoch,
                                       uint32_t wait_limit_us, const void* gate, void* out);

/* One split-KV decode step of this rank as ONE submission of the same two kernels as
 * tatara_attn_decode: the partitions of keys [key_begin, key_end) of this rank's cache slice, then
 * one merge kernel that (a) merges this rank's partitions to one record per head, (b) stores it into
 * slot `rank` of every rank's peer buffer (plain 8-byte peer stores over NVLink, each word carrying
 * {value, step number}, so no fence, flag or collective follows), (c) waits, bounded by
 * wait_limit_us (<= 2 000 000; on expiry nothing is written and tatara_ctx_sync returns
 * TATARA_DEVICE_WAIT_TIMEOUT), until the words of all `world` ranks carry this step's number and
 * (d) merges the world's records in rank order with the reference's combine
 * (src/backend/metal/kernels/attention.metal:1086-1108), gates and stores `out` on every rank --
 * the bits tatara_attn_combine gives on the gathered records.
 * peer_buffers: `world` device pointers, entry r = rank r's buffer of tatara_split_buffer_bytes(world)
 * zero-initialised bytes (tatara_peer_buffer_create / _open).  The step number lives on the device
 * and is advanced by the step itself, so no argument changes from token to token: the call may be
 * captured in a CUDA graph and replayed.  Every rank must issue the same sequence of steps, each
 * rank's kernels running at the same time as the others' (one process per GPU). */
uint64_t tatara_split_buffer_bytes(uint32_t world);
tatara_status tatara_attn_decode_split(tatara_ctx* ctx, void* stream, const void* q, const void* gate,
                                       const void* keys, const void* values, uint32_t key_begin,
                                       uint32_t key_end, uint32_t capacity, void* const* peer_buffers,
                                       uint32_t rank, uint32_t world, uint32_t wait_limit_us, void* out,
                                       void* scratch, uint64_t scratch_bytes);

/* Causal block prefill: slots 0 query, 1 K, 2 V, 3 gate, 4 out, 5 visible, 6 capacity,
 * 7 tile_rows, 8 tile_context (src/runtime/prefill_step.cpp:1661-1683).  Row r sits at
 * position context_base + r and attends keys 0..context_base + r of the lane cache (which
 * tatara_attn_qk_rope has filled). */
tatara_status tatara_attn_prefill(tatara_ctx* ctx, void* stream, const void* query,
                                  const void* gate, const void* keys, const void* values,
                                  uint32_t context_base, uint32_t rows, uint32_t capacity,
                                  void* out);

/* The numerical-control prefill family (attention_partial_blk + attention_combine_blk,
 * src/backend/metal/kernels/prefill_attention.metal:97-254): every row runs the decode
 * kernels' arithmetic.  Needs tatara_attn_decode_scratch_bytes(context_base+rows, rows). */
tatara_status tatara_attn_prefill_control(tatara_ctx* ctx, void* stream, const void* query,
                                          const void* gate, const void* keys, const void* values,
                                          uint32_t context_base, uint32_t rows, uint32_t capacity,
                                          void* out, void* scratch, uint64_t scratch_bytes);

/* ---- gated deltanet ------------------------------------------------------------------- */
/* gdn_prepare / gdn_conv_blk: slots 0 projection, 1 conv_in, 2 conv w, 3 qk, 4 value, 5 z,
 * 6 conv_out [, 7 rows] (src/runtime/decode_step.cpp:666-674, prefill_step.cpp:1936-1943). */
tatara_status tatara_gdn_prepare(tatara_ctx* ctx, void* stream, const void* projection,
                                 const void* conv_in, const void* conv_weights, void* qk,
                                 void* value, void* z, void* conv_out, uint32_t rows);

/* gdn_gates_blk: decay/beta planes [rows][32] f32
 * (src/backend/metal/kernels/prefill_gdn.metal:94-135). */
tatara_status tatara_gdn_gates(tatara_ctx* ctx, void* stream, const void* projection,
                               uint32_t projection_stride, const void* a_log, const void* dt_bias,
                               void* decay, void* beta, uint32_t rows);

/* gdn_recurrence: slots 0 qk, 1 value, 2 projection, 3 a_log, 4 dt_bias, 5 state_in, 6 y,
 * 7 state_out (src/runtime/decode_step.cpp:676-690).  state_in != state_out. */
tatara_status tatara_gdn_step(tatara_ctx* ctx, void* stream, const void* qk, const void* value,
                              const void* projection, const void* a_log, const void* dt_bias,
                              const void* state_in, void* y, void* state_out);

/* gdn_gate_norm(_blk): slots 0 y, 1 z, 2 norm w, 3 out (src/runtime/decode_step.cpp:692-697). */
tatara_status tatara_gdn_gate_norm(tatara_ctx* ctx, void* stream, const void* y, const void* z,
                                   const void* weight, void* out, uint32_t rows);

/* Lane-batched fused decode step (gdn_prepare_ms + gdn_recurrence_ms + gdn_gate_norm,
 * src/backend/metal/kernels/gdn.metal:231-378, src/runtime/decode_step.cpp:1037-1062):
 * one row per lane; conv and recurrent state live in pools addressed by the lane table.
 * Outputs: gated [lane][4096] bf16 (the o-proj input); y [lane][4096] bf16 optional. */
tatara_status tatara_gdn_decode_batch(tatara_ctx* ctx, void* stream, const void* projection,
                                      uint32_t projection_stride, const void* conv_weights,
                                      const void* a_log, const void* dt_bias,
                                      const void* norm_weight, void* conv_pool, void* rec_pool,
                                      const tatara_gdn_lane* lanes, uint32_t n_lanes, void* y,
                                      void* gated);

/* gdn_recurrence_gates_blk: slots 0 qk, 1 value, 2 decay, 4 beta, 5 state_in, 6 y,
 * 7 state_out, 8 rows (src/runtime/prefill_step.cpp:2003-2024).
 *   chunk == 64: chunked (WY / UT transform) evaluation of the same recurrence on the tensor
 *                cores; needs tatara_gdn_prefill_scratch_bytes(rows) bytes of scratch.
 *   chunk == 1 : the reference's own sequential scan (scratch may be NULL).
 * rows need not be a multiple of the chunk.  state_in != state_out. */
tatara_status tatara_gdn_prefill(tatara_ctx* ctx, void* stream, const void* qk, const void* value,
                                 const void* decay, const void* beta, const void* state_in,
                                 void* y, void* state_out, uint32_t rows, uint32_t chunk,
                                 void* scratch, uint64_t scratch_bytes);
uint64_t tatara_gdn_prefill_scratch_bytes(uint32_t rows);

/* ---- affine-Q4 projections on either side of the layers --------------------------------
 * The step before attn_qk_rope / gdn_prepare (hidden row -> projection row) and the step
 * after the gated output (attended / gated row -> hidden row).  Weights keep the reference's
 * layout: words [rows][k/8] u32 with nibble j of word w = column 8w + j, scales and biases
 * [rows][k/64] bf16 (group of 64 columns), w = q * scale + bias. */
typedef struct tatara_q4_matrix {
    const void* words;
    const void* scales;
    const void* biases;
    uint32_t rows; /* output columns this matrix contributes; a multiple of 16 */
    uint32_t reserved;
} tatara_q4_matrix;

/* Exact-row policy.  out[r][c] = bf16(q4_dot(input[r], row c)) with the reference's per-row
 * arithmetic sequence (q4_dot.metal:9-42; fused multiply-add chains, adjacent-pairs 32-lane
 * tree), so a row's bits do not depend on how many rows share the call: the row-batched and
 * block forms of the reference keep the same property (q4_dot.metal:44-104,
 * prefill_dense.metal:1-49).  The matrices' output columns are concatenated in order:
 *   attn_project  (attention.metal:1-41;  decode_step.cpp:705-711, prefill_step.cpp:1428):
 *                 {query+gate 8192, key 512, value 512}, k = 2048 -> projection[9216]
 *   gdn_project   (gdn.metal:1-46;        decode_step.cpp:657-664, prefill_step.cpp:1909-1915):
 *                 {qkv 8192, z 4096, b 32, a 32}, k = 2048 -> projection[12352]
 *   out_projection (gdn.metal:209-226;    decode_step.cpp:698-702, 732-736): one matrix of
 *                 2048 rows, k = 4096.
 * input [n_rows][input_stride] bf16, out [n_rows][out_stride] bf16 (strides in elements);
 * k a multiple of 512 and at most 6144 (four staged rows fit the default shared memory), at most
 * 4 matrices. */
tatara_status tatara_q4_project(tatara_ctx* ctx, void* stream, const void* input,
                                uint64_t input_stride, uint32_t n_rows,
                                const tatara_q4_matrix* matrices, uint32_t n_matrices, uint32_t k,
                                void* out, uint64_t out_stride);

/* Tensor-unit policy (the reference's QuantizedGemmPolicy::NativeDenseMma,
 * native_dense_qgemm.metal; prefill_step.cpp:1867-1907): weights are dequantised once to
 * bf16(q * scale + bias), [sum of rows][k], and block projections run as a bf16 GEMM with f32
 * accumulation on the tensor cores.  tatara_q4_dequantize is a load-time step; the result is
 * reused by every tatara_project_dense call. */
tatara_status tatara_q4_dequantize(tatara_ctx* ctx, void* stream, const tatara_q4_matrix* matrices,
                                   uint32_t n_matrices, uint32_t k, void* weights);
/* out[r][c] = bf16(sum_k input[r][k] * weights[c][k]); input [n_rows][input_stride], weights
 * [n][k] bf16, out [n_rows][out_stride].  k a multiple of 64, n a multiple of 32, strides
 * multiples of 8 elements, buffers 16-byte aligned. */
tatara_status tatara_project_dense(tatara_ctx* ctx, void* stream, const void* input,
                                   uint64_t input_stride, uint32_t n_rows, const void* weights,
                                   uint32_t n, uint32_t k, void* out, uint64_t out_stride);

/* ---- state snapshots --------------------------------------------------------------------
 * Device-to-device copy of a list of segments in one launch (all SMs, 32 KiB chunks dealt
 * round-robin).  Replaces the per-segment blit copies of the reference's prefix-state transfer
 * (src/runtime/prefix_state_transfer.cpp:236-262: one copy_buffer per segment between a decode
 * slot and the prefix-cache arena) and the per-head copies of its state record loader
 * (tools/native/decode_harness.cpp:339-461).  Addresses 16-byte aligned, lengths multiples of
 * 16 bytes; the whole list is validated before anything is enqueued; segments must not overlap
 * one another's destinations. */
typedef struct tatara_copy_segment {
    const void* src;
    void* dst;
    uint64_t bytes;
} tatara_copy_segment;
tatara_status tatara_state_copy(tatara_ctx* ctx, void* stream, const tatara_copy_segment* segments,
                                uint32_t n_segments);

/* ---- speculative-decode support: the GDN tape of a verify band and its replay -----------
 * A verify band of at most 16 rows runs the block kernels in their tape forms; after partial
 * acceptance the host restores the pre-band state and replays the committed rows
 * (src/engine/speculative_decode.cpp:517-596).  Tape geometry is the reference's
 * (tools/generate_kernel_library.py:2045-2049): 40 layers x 16 rows;
 *   tape      f32: delta [layer][row][32][128] | key [layer][row][16][128] | gates [layer][row][32][2]
 *   conv_tape bf16: [layer][row][3][8192], the conv tail after each row.
 * Unlike the reference kernels, which silently skip the tape when rows > 16, these reject it. */
uint64_t tatara_gdn_tape_bytes(void);
uint64_t tatara_gdn_conv_tape_bytes(void);
/* gdn_conv_tape_blk: tatara_gdn_prepare plus slots 8 conv_tape, 9 tape_layer
 * (src/backend/metal/kernels/prefill_gdn.metal:322-420; src/runtime/prefill_step.cpp:1931-1946). */
tatara_status tatara_gdn_prepare_tape(tatara_ctx* ctx, void* stream, const void* projection,
                                      const void* conv_in, const void* conv_weights, void* qk,
                                      void* value, void* z, void* conv_out, uint32_t rows,
                                      void* conv_tape, uint32_t tape_layer);
/* gdn_recurrence_gates_tape_blk: the sequential scan of tatara_gdn_prefill (chunk 1) plus slots
 * 9 tape, 10 tape_layer (prefill_gdn.metal:434-527; prefill_step.cpp:2003-2028). */
tatara_status tatara_gdn_prefill_tape(tatara_ctx* ctx, void* stream, const void* qk,
                                      const void* value, const void* decay, const void* beta,
                                      const void* state_in, void* y, void* state_out, uint32_t rows,
                                      void* tape, uint32_t tape_layer);
/* gdn_tape_replay_blk: slots 0 tape, 1 state_in, 2 state_out, 3 steps, 4 tape_layer
 * (prefill_gdn.metal:529-569; speculative_decode.cpp:546-555).  state_out has the bits the
 * taped scan itself reaches after `steps` rows; steps == 0 copies the state. */
tatara_status tatara_gdn_tape_replay(tatara_ctx* ctx, void* stream, const void* tape,
                                     const void* state_in, void* state_out, uint32_t steps,
                                     uint32_t tape_layer);

/* ---- lane tables in device memory (CUDA-graph replay of a decode token) ------------------
 * The reference re-encodes a command buffer per token with the stream group's contexts and state
 * slots as constants (src/runtime/decode_step.cpp:1002-1426, tools/native/tatara_serve.cpp:
 * 1463-1777).  Here the same tables may live in DEVICE memory: nothing about a token is then a
 * kernel argument, so a token's launches can be captured once into a CUDA graph and replayed for
 * every token, with tatara_lanes_advance (context + 1; gated-delta in / out offsets swapped) as
 * the node between tokens.  Same kernels, same per-lane cut, same output bits as the host-table
 * entry points.  What the host cannot check any more is checked on the device: a context beyond
 * the capacity reads and writes nothing for that lane and latches TATARA_CONTEXT_OUT_OF_RANGE
 * for the next tatara_ctx_sync.  `scratch` must hold tatara_attn_decode_scratch_bytes(capacity,
 * n_lanes).  The calls of one context share one schedule buffer: use one stream per context. */
tatara_status tatara_attn_qk_rope_batch_indirect(tatara_ctx* ctx, void* stream, const void* projection,
                                                 const void* q_weight, const void* k_weight,
                                                 void* q_out, void* gate_out, void* keys_pool,
                                                 void* values_pool, uint32_t capacity,
                                                 const tatara_attn_lane* lanes_device,
                                                 uint32_t n_lanes, uint32_t projection_stride,
                                                 uint32_t query_stride);
tatara_status tatara_attn_decode_batch_indirect(tatara_ctx* ctx, void* stream, const void* q,
                                                const void* gate, const void* keys_pool,
                                                const void* values_pool,
                                                const tatara_attn_lane* lanes_device, uint32_t n_lanes,
                                                uint32_t capacity, uint32_t query_stride, void* out,
                                                void* scratch, uint64_t scratch_bytes);
tatara_status tatara_gdn_decode_batch_indirect(tatara_ctx* ctx, void* stream, const void* projection,
                                               uint32_t projection_stride, const void* conv_weights,
                                               const void* a_log, const void* dt_bias,
                                               const void* norm_weight, void* conv_pool,
                                               void* rec_pool, const tatara_gdn_lane* lanes_device,
                                               uint32_t n_lanes, void* y, void* gated);
tatara_status tatara_lanes_advance(tatara_ctx* ctx, void* stream, tatara_attn_lane* attn_lanes_device,
                                   uint32_t n_attn, tatara_gdn_lane* gdn_lanes_device, uint32_t n_gdn);

#ifdef __cplusplus
}
#endif
#endif /* TATARA_B200_H_ */
