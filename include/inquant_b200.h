/*
 * C ABI of libinquant_b200.so -- the B200 (sm_100a) implementation of the InQuant
 * packed-KV hot path.  Plain pointers and sizes only; every pointer is a DEVICE pointer
 * unless its comment says "host".  Every call enqueues work on `stream` and returns
 * without synchronising; the return value is INQ_OK or a negative INQ_ERR_* code for
 * arguments rejected on the host (nothing is launched in that case).  Data-dependent
 * failures (non-finite input, a device-side wait that ran out) are reported through the
 * caller's 32-bit device status word, which kernels only ever OR bits into.
 *
 * Each entry point names the reference interface (file:line in
 * changzihan22/InQuant-open-source) whose work it performs.
 */
#ifndef INQUANT_B200_H
#define INQUANT_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef void* inq_stream_t; /* a cudaStream_t */

enum {
  INQ_OK = 0,
  INQ_ERR_ARGUMENT = -1,    /* shape / stride / enum outside the supported set */
  INQ_ERR_UNSUPPORTED = -2, /* valid for the reference, not built for this size */
  INQ_ERR_CUDA = -3,        /* a CUDA runtime call failed; see inq_last_error() */
  INQ_ERR_CAPACITY = -4     /* exceeds a fixed capacity stated by the entry point */
};

enum { INQ_F32 = 0, INQ_F16 = 1, INQ_BF16 = 2 };

/* bits of the device status word */
enum {
  INQ_STATUS_NONFINITE = 1,       /* input (or a stored fp16 parameter) was not finite */
  INQ_STATUS_BAD_INDEX = 2,       /* a role-map entry, tail position or (when the caller passed the
                                   * pool size) page id was out of range and was not used */
  INQ_STATUS_WAIT_TIMEOUT = 4     /* a bounded device-side wait gave up */
};

/* Human-readable text of the last INQ_ERR_CUDA on this thread (host pointer, static). */
const char* inq_last_error(void);
int inq_version(void);

/* ---------------------------------------------------------------- addressing helpers
 * Inputs are 4-D logical tensors [outer, inner, tokens, channels] with unit channel
 * stride; strides are in ELEMENTS.  This covers [batch, heads, T, C] tensors, a temporal
 * block axis moved into `outer` (reference cache.py:104-107) and the token-major
 * [tokens, heads, C] layout of the paged backend (reference backend.py:146-147).
 *
 * Outputs are addressed per row (outer index p, inner index h) as
 *     base + slot(p) * outer_stride_bytes + h * inner_stride_bytes,
 * slot(p) = page_ids ? page_ids[p] : p.  A compact tensor uses the obvious strides; a
 * physical page pool uses outer_stride_bytes = page_bytes for every field.
 */
typedef struct {
  void* base;            /* NULL = field not wanted */
  int64_t outer_stride;  /* bytes */
  int64_t inner_stride;  /* bytes */
} inq_field_t;

typedef struct {
  const void* x;         /* input elements of type `dtype` */
  int32_t dtype;         /* INQ_F32 / INQ_F16 / INQ_BF16 */
  int64_t n_outer, n_inner;
  int64_t stride_outer, stride_inner, stride_token; /* elements */
  int32_t tokens, channels;
  const void* page_ids;  /* optional [n_outer] physical slots; NULL = identity */
  int32_t page_ids_i64;  /* 1 if page_ids is int64, 0 if int32 */
  int64_t num_slots;     /* slots the destination holds: a row whose page id lies outside
                          * [0, num_slots) is not written and INQ_STATUS_BAD_INDEX is set;
                          * 0 = the caller vouches for the ids (they are not checked) */
} inq_input_t;

/* ---------------------------------------------------------------- K4 encoder
 * Fused sampled-saliency statistics, donor selection and mixed 4/8-bit key packing for
 * every (outer, inner) row independently.
 * Replaces: codec.py:181-243 `quantize` (statistics :202-210, `_reuse_map` :137-178,
 * scales :218-221, codes/pack :223-233), triton_selection.py:11-60 `_select`/`reuse_map`,
 * and the per-block export of cache.py:89-119 `_quantize_temporal_blocks`; with a page
 * pool as destination also layout.py:103-115 `pack_pages_into` and packing.py:7-55.
 *   count           floor(channels * salient_fraction), 0..channels/2
 *   min_error       1 = donor pool restricted by full-block reconstruction error
 *   payload         u8 [T, C/2] per row;  scales f32 [C];  padding f32 [count]
 *   salient/donors  descriptor lists [count], u8 or i32 (`descriptor_i32`)
 *   roles           optional per-channel role map [C], `role_bytes` = 1 (int8,
 *                   triton_attention.py:301-309) or 2 (int16, layout.py:73-77)
 * Requirements: channels even, <= 1024; tokens >= 1; sample_stride >= 1.
 */
typedef struct {
  inq_input_t in;
  int32_t sample_stride, count, min_error;
  inq_field_t payload, scales, salient, donors, padding, roles;
  int32_t descriptor_i32, role_bytes;
} inq_k4_encode_args_t;
int inq_k4_encode(const inq_k4_encode_args_t* args /* host */, int32_t* status, inq_stream_t stream);

/* Stand-alone donor selection on precomputed statistics.
 * Replaces: codec.py:137-178 `_reuse_map`, triton_selection.py:46-60 `reuse_map`.
 * saliency / donor_error: f32 [rows, channels] (donor_error may be NULL);
 * sources / donors: int64 [rows, count]. */
int inq_select_donors(const float* saliency, const float* donor_error, int64_t rows, int32_t channels,
                      int32_t count, int64_t* sources, int64_t* donors, inq_stream_t stream);

/* Sampled statistics alone (used by stage-by-stage benchmarks and tests).
 * Replaces: codec.py:202-210.  Outputs f32 [rows, C]; any may be NULL. */
int inq_k4_statistics(const inq_input_t* in /* host */, int32_t sample_stride, float* saliency,
                      float* sampled_mean, float* donor_error, float* absmax, inq_stream_t stream);

/* Exact inverse of the K4 layout.  Replaces: codec.py:112-134 `PackedTensor.dequantize`.
 * All tensors compact: payload [rows,T,C/2], scales [rows,C], lists [rows,count]. */
int inq_k4_dequantize(const uint8_t* payload, const float* scales, const void* salient, const void* donors,
                      int32_t descriptor_i32, const float* padding, int64_t rows, int32_t tokens,
                      int32_t channels, int32_t count, void* out, int32_t out_dtype, inq_stream_t stream);
/* The same with rows (outer, inner) written at out + outer * out_stride_outer + inner *
 * out_stride_inner (elements; a row's tokens stay contiguous): the blocks of one encoder launch,
 * [blocks, heads, T, C], land directly in a [heads, tokens, C] history at their token positions.
 * Replaces: the per-block dequantize + torch.cat of cache.py:328-345 `materialize`. */
int inq_k4_dequantize_strided(const uint8_t* payload, const float* scales, const void* salient, const void* donors,
                              int32_t descriptor_i32, const float* padding, int64_t rows_outer, int32_t rows_inner,
                              int32_t tokens, int32_t channels, int32_t count, void* out, int64_t out_stride_outer,
                              int64_t out_stride_inner, int32_t out_dtype, inq_stream_t stream);

/* ---------------------------------------------------------------- V encoder
 * Per-token, per-group affine INT2/INT4 with fp16 scale and minimum.
 * Replaces: value_codec.py:51-72 `quantize_values`, :75-88 `quantize_value_blocks`.
 *   payload u8 [T, C*bits/8]; scales/offsets f16 [T, C/group] per row.
 * Requirements: bits 2|4, group 32|64|128, channels % group == 0, channels <= 256. */
typedef struct {
  inq_input_t in;
  int32_t bits, group;
  inq_field_t payload, scales, offsets;
} inq_v_encode_args_t;
int inq_v_encode(const inq_v_encode_args_t* args /* host */, int32_t* status, inq_stream_t stream);

/* Replaces: value_codec.py:38-48 `PackedValues.dequantize`. */
int inq_v_dequantize(const uint8_t* payload, const void* scales, const void* offsets, int64_t rows,
                     int32_t tokens, int32_t channels, int32_t bits, int32_t group, void* out,
                     int32_t out_dtype, inq_stream_t stream);
/* Strided destination as in inq_k4_dequantize_strided. */
int inq_v_dequantize_strided(const uint8_t* payload, const void* scales, const void* offsets, int64_t rows_outer,
                             int32_t rows_inner, int32_t tokens, int32_t channels, int32_t bits, int32_t group, void* out,
                             int64_t out_stride_outer, int64_t out_stride_inner, int32_t out_dtype, inq_stream_t stream);

/* Role maps from descriptor lists.  Replaces: triton_attention.py:301-309 `_write_maps`
 * and the map construction inside packing.py:24-29.  lists [rows,count] u8 or i32. */
int inq_build_roles(const void* salient, const void* donors, int32_t descriptor_i32, int64_t rows,
                    int32_t channels, int32_t count, void* roles, int32_t role_bytes, inq_stream_t stream);

/* Scatter of already-encoded codec output (compact tensors [pages, kv_heads, ...] as inq_k4_encode /
 * inq_v_encode write them, 16 salient channels, V2 in groups of 64) into the physical pages
 * page_ids[p] of a pool in the serving layout (layout.py:18-42), building each page's int16 role
 * map on the way; one launch.  page_offsets as in inq_decode_args_t.  Every pointer, page_bytes and
 * every offset must be a multiple of 16.  A page id outside [0, num_slots) is not written and sets
 * INQ_STATUS_BAD_INDEX (num_slots 0: ids are not checked).
 * Replaces: inquant_vllm/packing.py:7-55 `_write_pages` / `write_codec_pages`. */
typedef struct {
  const uint8_t* key_payload; const float* key_scales; const uint8_t* salient; const uint8_t* donors;
  const float* key_padding; const uint8_t* value_payload; const void* value_scales; const void* value_offsets;
  int64_t pages;
  int32_t heads, block_tokens, count;
  uint8_t* pool;
  int64_t page_bytes;
  int64_t page_offsets[6];
  const void* page_ids;
  int32_t page_ids_i64;
  int64_t num_slots;
  int32_t* status;
} inq_write_pages_args_t;
int inq_write_codec_pages(const inq_write_pages_args_t* args /* host */, inq_stream_t stream);

/* ---------------------------------------------------------------- decode attention
 * One decode step of single-query grouped-query attention over packed K4/V2 history plus
 * the exact sink and recent tail, for one sequence (a layer of a request) or a batch of
 * them in ONE launch; split-KV partials are merged inside the same launch.
 * Replaces: triton_attention.py:67-181 `_attention_partials` + `_reduce_partials` as
 * launched by `PackedDecodeState.decode` (:317-388), and inquant_vllm/kernels.py:8-88
 * `_paged_partials` / `paged_decode`.
 *
 * layout 0 ("table", triton_attention.py:277-295): block i is reached through six device
 *   pointers table[i][0..5] = key payload, key scales, key padding, value payload, value
 *   scales, value offsets, each a compact [kv_heads, ...] tensor; roles is the int8 map
 *   [n_blocks, kv_heads, 128] of triton_attention.py:301-309.
 * layout 1 ("paged", layout.py:18-42): block i is page page_table[i] of `pool`;
 *   page_offsets = byte offsets of key_scales, key_map, key_padding, value_payload,
 *   value_scales, value_offsets inside a page.
 * Requirements: head_dim 128, V2 with group 64, query dtype fp16 or bf16 (the dense sink
 * and tail share it), dense rows 16-byte aligned.  Masks: packed tokens whose position in
 * the sequence (block*block_tokens + t) is below first_visible are skipped (the exact sink
 * replaces them, kernels.py:41); the first tail_skip tail tokens are skipped (kernels.py:53).
 */
typedef struct {
  const void* query;             /* [q_heads, 128], head stride query_head_stride elements */
  void* output;                  /* [q_heads, 128] contiguous, query dtype */
  int64_t query_head_stride;
  const int64_t* table;          /* layout 0 */
  const int8_t* roles;           /* layout 0 */
  const uint8_t* pool;           /* layout 1 */
  const int32_t* page_table;     /* layout 1 */
  const void* sink_key; const void* sink_value; const void* tail_key; const void* tail_value;
  int64_t sink_key_stride_h, sink_key_stride_t, sink_value_stride_h, sink_value_stride_t;   /* elements */
  int64_t tail_key_stride_h, tail_key_stride_t, tail_value_stride_h, tail_value_stride_t;
  int32_t n_blocks, sink_tokens, tail_tokens, first_visible, tail_skip;
  int32_t pool_pages;     /* layout 1: pages in `pool`.  A page_table entry outside [0, pool_pages)
                           * is never dereferenced: page 0 is read in its place and
                           * INQ_STATUS_BAD_INDEX is set (the step's output is then meaningless);
                           * 0 = the caller vouches for the table (entries are not checked) */
  const int32_t* tail_tokens_device; /* optional: overrides tail_tokens, read on the device */
  float* partial_output;  /* optional [q_heads][130] fp32: when set, `output` is not written; the
                           * un-normalised record (acc[128], m in base-2 units, l) of each query
                           * head is stored instead -- the reference's partial format
                           * (triton_attention.py:162-165) -- for a cross-GPU merge */
  /* The step's new token, used only by launches with `fused_append` set (else ignored): rows
   * [kv_heads][128] of the query dtype, 16-byte aligned, `new_stride_h` elements apart.  The launch
   * attends to the token as position tail_tokens of the tail (tail_tokens counts the tokens BEFORE
   * it), stores it at that position of tail_key / tail_value (position >= tail_capacity: not
   * stored, INQ_STATUS_BAD_INDEX) and, once every CTA has read the length, adds one to
   * *tail_tokens_device.  Replaces the separate inq_append_token_batch launch of a decode step
   * (cache.py:256-259, 271-299; backend.py:158-163). */
  const void* new_key; const void* new_value;
  int64_t new_stride_h;
  int32_t tail_capacity;
  int32_t reserved;
  const int8_t* value_roles;  /* layout 0 with value_kind 1: role map of the value blocks, int8
                               * [n_blocks][kv_heads][128], as `roles` is for the keys */
} inq_decode_seq_t;

/* Split-KV across the GPUs of one node inside the decode launch itself (no counterpart in the
 * reference, which is single-GPU): the CTA that merges this rank's parts of a pair
 * (sequence, KV head, tile of 8 query heads) stores the pair's un-normalised record straight into
 * every peer's inbox over NVLink peer memory, waits for the peers' records of the same pair in its
 * own inbox -- a bounded wait: after `spin_limit` polls it sets INQ_STATUS_WAIT_TIMEOUT and writes
 * zero rows -- and merges all records in rank order (the cross-rank form of
 * triton_attention.py:168-181), so every rank writes the same `output`.  Every 32-bit word of a
 * record travels as one indivisible 8-byte store {word, step number}; a reader takes a word when its
 * step number is the current one, so the launch needs neither a system-scope fence nor flag words.
 * An inbox holds inq_decode_exchange_inbox_bytes(world, n_rows) bytes, zeroed before the first step
 * (inq_peer_buffer_create / _open); one inbox serves either inq_exchange_merge or this form, not
 * both.  Every rank launches the same steps in the same order; the launch needs all its CTAs
 * resident (it always sizes its grid so) and other work on the GPU only delays the wait.  The struct
 * lives in DEVICE memory. */
typedef struct {
  void* inboxes[8];       /* inbox of every rank as mapped into this process; [rank] is the own one */
  int32_t* epoch;         /* device, zero before the first step: [0] = steps completed, advanced by the launch */
  int64_t n_rows;         /* n_seq * kv_heads * q_per_kv, the same on every rank */
  int32_t world, rank;
  int32_t spin_limit;     /* polls of >= 100 ns before a wait gives up; 0 = default (a fraction of a second) */
  int32_t reserved;
} inq_decode_exchange_t;

typedef struct {
  int32_t n_seq;
  const inq_decode_seq_t* seqs_device; /* [n_seq] in device memory, or NULL when n_seq == 1 */
  const inq_decode_seq_t* seq_host;    /* host: the single sequence when seqs_device is NULL */
  int32_t kv_heads, q_per_kv, block_tokens, n_pad; /* n_pad = salient channels per head */
  int32_t layout, dtype;
  float scale;
  int64_t page_bytes;
  int64_t page_offsets[6];
  /* Work is balanced over the whole batch: the packed slices of all pairs
   * (sequence, KV head, tile of 8 query heads), in that order, form one list that is cut into
   * equal ranges, one per resident CTA.  pair_starts[p] = sum of inq_decode_units(n_blocks of
   * the pair's sequence, block_tokens) over pairs before p; [n_pairs + 1] int64 in DEVICE
   * memory.  NULL is allowed when every sequence holds `uniform_blocks` blocks (with
   * seq_host the count is taken from the descriptor). */
  const int64_t* pair_starts;
  int64_t total_units;      /* pair_starts[n_pairs]; ignored without pair_starts */
  int32_t uniform_blocks;
  float* partials;          /* scratch, contents undefined on entry and exit */
  int64_t partials_floats;  /* its size: at least inq_decode_workspace_floats(n_pairs, total_units) */
  int32_t* counters;        /* scratch: n_pairs + 1 ints, ZERO on entry, left zero on exit */
  int32_t* status;          /* device status word */
  int32_t fused_append;     /* 1: every sequence's new_key / new_value token is appended by this launch */
  const inq_decode_exchange_t* exchange_device; /* optional, DEVICE memory: exchange and merge the records of
                                                 * every pair with the peer GPUs inside this launch;
                                                 * `partial_output` of the sequences is then ignored */
  int32_t value_kind;       /* 0: values as 2-bit codes in groups of 64 channels (value_codec.py);
                             * 1: values stored as InQuant packed tensors like the keys (the reference's
                             *    CacheConfig default, value_bits=None): table columns 3..5 then hold the
                             *    value payload [kv_heads][tokens][64], scales fp32 [kv_heads][128] and
                             *    padding fp32 [kv_heads][16]; served for layout 0, n_pad 16 on both sides
                             *    and blocks of a multiple of 32 tokens (>= 64), else INQ_ERR_UNSUPPORTED
                             *    (inq_decode_generic serves the rest);
                             * 2: values as 4-bit codes with fp16 scale and offset per token and group of
                             *    128 / value_groups channels (value_codec.py with bits=4): table columns 3..5
                             *    hold payload [kv_heads][tokens][64], scales and offsets
                             *    [kv_heads][tokens][value_groups]; same geometry limits as kind 1 */
  int32_t value_groups;     /* kind 2: 1, 2 or 4 (groups of 128, 64 or 32 channels); kind 0: 0 or 2 for the
                             * groups of 64 channels, 1 for one group of 128, 4 for groups of 32 (geometry limits
                             * of kind 1) */
} inq_decode_args_t;
int inq_decode_attention(const inq_decode_args_t* args /* host */, inq_stream_t stream);
/* The same decode step for callers that cannot allocate device memory (a serving engine that
 * has committed the whole device to its own page pool, a host runtime that owns all device
 * memory).  It has no counterpart in the reference.  The
 * partial records and arrival counters live in a fixed array inside the library (about 4.2 MB
 * per device, held until the process exits), so `partials`, `partials_floats` and `counters` of
 * the arguments are ignored.  Limits: at most 256 pairs (n_seq * kv_heads * ceil(q_per_kv/8))
 * and at most 1024 partial records (resident CTAs + pairs) per launch; larger launches return
 * INQ_ERR_CAPACITY.  It calls no cudaMalloc/cudaFree.  The first call on a device resolves the
 * array's address and zeroes its counters on `stream`.
 * All calls on a device share the array: launches that may overlap on the GPU (different
 * streams) race on it; calls on one stream do not. */
int inq_decode_attention_noalloc(const inq_decode_args_t* args /* host */, inq_stream_t stream);
/* Log-sum-exp merge of partial records from n_parts ranks (split-KV of one long sequence over
 * GPUs): records [n_parts][n_rows][130] fp32 as written through `partial_output`, out
 * [n_rows][128] fp16/bf16.  Replaces: triton_attention.py:168-181 `_reduce_partials` applied
 * across ranks after an all-gather. */
int inq_merge_partials(const float* records, int32_t n_parts, int64_t n_rows, void* out, int32_t out_dtype,
                       inq_stream_t stream);
/* Every sealed block of one cached layer back into dense key and value histories in ONE launch, addressed
 * through the layer's decode descriptors (the 6-pointer block table and the int8 role map of
 * inq_decode_seq_t, layout 0): what InQuantCache.materialize (cache.py:328-345) does block by block
 * with PackedTensor.dequantize (codec.py:112-134) and PackedValues.dequantize (value_codec.py:43-48),
 * same arithmetic, same rounding.  K4 keys with `count` salient channels and 2-bit values in groups of
 * 64, 128 channels; rows of head h land at out + h * stride_h + (position + block * tokens + t) * 128
 * elements of out_dtype (fp16 / bf16); out pointers 16-byte aligned, stride_h a multiple of 8. */
int inq_restore_blocks_table(const int64_t* table, const int8_t* roles, int32_t n_blocks, int32_t heads, int32_t tokens,
                             int32_t count, void* out_key, void* out_value, int64_t stride_h, int64_t position,
                             int32_t out_dtype, inq_stream_t stream);

/* Split-KV across the GPUs of ONE node without a library collective: exchange of the partial
 * records over NVLink peer memory fused with their merge, one launch per rank and decode step.
 * Every rank owns an inbox (inq_peer_buffer_create, inq_exchange_inbox_bytes bytes, zeroed) that
 * every other process maps (inq_peer_buffer_open).  The kernel stores this rank's records into
 * all peers' inboxes, publishes a per-chunk step flag with a release store, waits -- bounded --
 * for the peers' flags in its own inbox and merges as inq_merge_partials does.  All ranks must
 * launch it the same number of times; `epoch` (device int32[2], zeroed once, owned by the kernel)
 * counts the steps.  A wait that runs out sets INQ_STATUS_WAIT_TIMEOUT in `status`, zeroes the
 * affected output rows and returns.  At most 8 ranks; INQ_ERR_CAPACITY when the CTAs of a launch
 * could not all be resident.  With n_local == world the entries of `ranks` are ALL ranks, emulated
 * inside one cooperative grid on the current device (for tests on a single GPU).
 * Replaces: nothing in the reference (it has no multi-GPU path); the merge is
 * triton_attention.py:168-181 `_reduce_partials` applied across ranks. */
typedef struct {
  const float* local;     /* device: this rank's records [n_rows][130] fp32 (partial_output) */
  void* const* inboxes;   /* HOST array [world]: the inbox of every rank as mapped here (own included) */
  void* out;              /* device: [n_rows][128] fp16/bf16 */
  int32_t* epoch;         /* device int32[2] */
  int32_t* status;        /* device status word */
  int32_t rank;
} inq_exchange_rank_t;
typedef struct {
  const inq_exchange_rank_t* ranks;  /* host: 1 entry (this process), or `world` entries to emulate */
  int32_t n_local;                   /* 1 or world */
  int32_t world;
  int64_t n_rows;
  int32_t out_dtype;                 /* INQ_F16 or INQ_BF16 */
  int32_t spin_limit;                /* polls (>= 100 ns each) before a wait gives up; 0 = default (~0.3 s) */
} inq_exchange_args_t;
int inq_exchange_merge(const inq_exchange_args_t* args /* host */, inq_stream_t stream);
int64_t inq_exchange_inbox_bytes(int32_t world, int64_t n_rows);
int64_t inq_decode_exchange_inbox_bytes(int32_t world, int64_t n_rows);   /* inbox of inq_decode_exchange_t */
/* Device memory other processes of the node can map: create = cudaMalloc + zero fill + a 64-byte
 * CUDA IPC handle to send to the peers; open maps a peer's buffer (enabling peer access);
 * close / destroy undo open / create.  These four calls synchronise with the device. */
int inq_peer_buffer_create(int64_t bytes, void** ptr, unsigned char* handle /* 64 bytes out */);
int inq_peer_buffer_open(const unsigned char* handle /* 64 bytes */, void** ptr);
int inq_peer_buffer_close(void* ptr);
int inq_peer_buffer_destroy(void* ptr);
/* Packed decode attention for codec variants outside the K4/V2 preset (slower, general): values
 * stored as InQuant packed tensors (value_kind 1: table columns 3..5 are payload, f32 scales, f32
 * padding, with an int8 role map like the keys') or as 2/4-bit groups of `value_group` channels
 * (value_kind 0: payload, f16 scales, f16 offsets); fp32, fp16 or bf16 queries with sink/tail in
 * the same dtype; even head dimensions up to 256.  One sequence, table layout as in
 * inq_decode_seq_t.  `partials` is scratch of inq_decode_generic_workspace_floats floats.
 * Replaces: triton_attention.py:67-181 for `value_bits=None`, V4, value groups of 32/128 and
 * fp32 queries (triton_attention.py:122-124, tests/test_triton_attention.py:23-25). */
typedef struct {
  const void* q;              /* [kv_heads * q_per_kv][head_dim] rows, `q_stride_h` elements apart */
  void* out;                  /* [kv_heads * q_per_kv][head_dim], contiguous */
  int64_t q_stride_h;
  const int64_t* table;       /* device: [n_blocks][6] pointers */
  const int8_t* key_roles;    /* device: [n_blocks][kv_heads][head_dim] */
  const int8_t* value_roles;  /* device, value_kind 1 only */
  const void *sink_key, *sink_value, *tail_key, *tail_value;
  int64_t sink_key_stride_h, sink_key_stride_t, sink_value_stride_h, sink_value_stride_t;
  int64_t tail_key_stride_h, tail_key_stride_t, tail_value_stride_h, tail_value_stride_t;
  int32_t n_blocks, sink_tokens, tail_tokens;
  int32_t kv_heads, q_per_kv, block_tokens, head_dim, key_pad, value_pad;
  int32_t value_kind, value_bits, value_group;
  int32_t dtype;              /* INQ_F32 / INQ_F16 / INQ_BF16: query, output, sink and tail */
  float scale;
  float* partials;
  int64_t partials_floats;
} inq_decode_generic_args_t;
int inq_decode_generic(const inq_decode_generic_args_t* args /* host */, inq_stream_t stream);
int64_t inq_decode_generic_workspace_floats(int32_t q_heads, int32_t n_blocks, int32_t sink_tokens,
                                            int32_t tail_tokens, int32_t head_dim);

/* Chunked-prefill attention on tcgen05 tensor cores with TMEM accumulators: causal attention of
 * `q_tokens` new query tokens over `kv_tokens` keys and values, where the last `q_tokens` rows of
 * k/v are the chunk's own tokens and the rows before them the history (for a packed cache: the
 * exact sink, the dequantised blocks written by inq_k4_dequantize / inq_v_dequantize, and the
 * exact tail).  Query i attends to rows 0 .. kv_tokens - q_tokens + i.  Layouts: q/out
 * [q_heads][q_tokens][128], k/v [kv_heads][kv_tokens][128], fp16 or bf16, element strides below
 * (multiples of 8, bases 16-byte aligned); head dimension 128; q_heads a multiple of kv_heads.
 * Replaces: cache.py:179-200 `update` returning the materialised history to the model's SDPA call
 * (qwen_fused.py:112-121, the original forward) for query chunks after the first. */
typedef struct {
  const void* q;
  const void* k;
  const void* v;
  void* out;
  int64_t q_stride_h, q_stride_t, k_stride_h, k_stride_t, v_stride_h, v_stride_t, o_stride_h, o_stride_t;
  int32_t q_heads, kv_heads, q_tokens, kv_tokens;
  int32_t dtype;              /* INQ_F16 or INQ_BF16 */
  float scale;                /* softmax scale */
  int32_t* status;            /* device status word (INQ_STATUS_WAIT_TIMEOUT on a stuck barrier) */
  void* workspace;            /* optional device scratch: lets the kernel cut the KV range of every */
  int64_t workspace_bytes;    /* (256 rows, head) item into segments that fill the SMs evenly      */
} inq_prefill_args_t;
int inq_prefill_attention(const inq_prefill_args_t* args /* host */, inq_stream_t stream);
/* Scratch that allows every cut inq_prefill_attention may choose. */
int64_t inq_prefill_workspace_bytes(int32_t q_heads, int32_t q_tokens);
/* Work units (32-token slices, at least 1) of one pair whose sequence holds n_blocks blocks. */
int64_t inq_decode_units(int32_t n_blocks, int32_t block_tokens);
/* Scratch floats that suffice for a launch with n_pairs pairs and total_units work units on
 * the current device. */
int64_t inq_decode_workspace_floats(int32_t n_pairs, int64_t total_units);

/* ---------------------------------------------------------------- incremental append
 * Writes the key and value rows of ONE new token (all KV heads) at `tail_position` of the
 * exact recent tail and, while the attention sink is still filling (sink_position >= 0),
 * into the sink as well.  With `tail_counter` the position is read from that device int
 * and incremented by the kernel, so a decode loop needs no host round trip.
 * Replaces: the per-token `torch.cat` + `clone` of cache.py:256-259, 271-299 and the tail
 * writes of backend.py:158-163.  Strides and row_bytes are BYTES, multiples of 16. */
typedef struct {
  const void* key; const void* value; int64_t src_stride_h;  /* new token rows, [heads, row] */
  void* tail_key; void* tail_value; int64_t tail_stride_h, tail_stride_t;
  int32_t tail_position, tail_capacity;
  int32_t* tail_counter;          /* optional device position, overrides tail_position */
  void* sink_key; void* sink_value; int64_t sink_stride_h, sink_stride_t;
  int32_t sink_position;          /* < 0: sink already full */
  int32_t heads, row_bytes;
  int32_t* status;
} inq_append_args_t;
int inq_append_token(const inq_append_args_t* args /* host */, inq_stream_t stream);
/* The same for `count` independent sequences (one layer of one request each) in one launch;
 * the records live in DEVICE memory and must satisfy the alignment rules above (they are
 * not re-checked); their `status` field is ignored in favour of the argument. */
int inq_append_token_batch(const inq_append_args_t* records_device, int32_t count, int32_t* status,
                           inq_stream_t stream);

/* ---------------------------------------------------------------- sealing blocks in one call
 * Everything a cache update that seals blocks does on the device, issued by ONE host call on one
 * stream: the key encoder, the value encoder (`value_k4` when values are stored as InQuant tensors,
 * `value` for the affine 2/4-bit codec; either may be NULL) and up to four dense row-range copies
 * (the tokens the attention sink takes, the remainder that becomes the new exact tail; source and
 * destination are [heads, tokens, row_bytes] with the byte strides given, all multiples of 16, and
 * must not overlap).  All arguments are checked before the first launch.
 * Replaces: cache.py:271-306 (`_append`: cat, one codec call per temporal block through
 * cache.py:89-119 / value_codec.py:75-88, cloned sink and tail) as one host call. */
typedef struct {
  const void* src; void* dst;
  int64_t src_stride_h, src_stride_t, dst_stride_h, dst_stride_t;   /* bytes */
  int32_t tokens;       /* rows per head; 0: entry unused */
  int32_t reserved;
} inq_row_copy_t;
typedef struct {
  const inq_k4_encode_args_t* key;        /* NULL: no key encoder launch */
  const inq_k4_encode_args_t* value_k4;   /* NULL: values are not InQuant tensors */
  const inq_v_encode_args_t* value;       /* NULL: no affine value encoder launch */
  inq_row_copy_t copies[4];
  int32_t n_copies, heads, row_bytes, reserved;
} inq_seal_args_t;
int inq_seal_blocks(const inq_seal_args_t* args /* host */, int32_t* status, inq_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* INQUANT_B200_H */
