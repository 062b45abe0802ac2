// Single-query grouped-query attention over the packed K4/V2 history plus the exact
// (bf16/fp16) sink and recent tail, with the split-KV partials merged by the last CTA of
// every (sequence, KV head, 8-query-head tile) pair -- one launch per decode step, for one
// layer or for a batch of (request, layer) sequences.
//
// Work decomposition.  The 32-token packed slices of all pairs form one flat list that is cut
// into gridDim.x equal ranges (the grid is SMs x resident CTAs); a CTA walks its range pair by
// pair and its four warps cut each segment again.  Every pair also occupies a few list positions
// without slices (its ramp): they stand for the fixed cost of visiting a pair, so that a CTA
// whose range crosses a pair boundary receives fewer slices.  Blocks of at most 16 tokens
// (16-token pages) use a variant of the kernel with 16-token slices that carry their block's
// metadata in the slice's own ring stage.  The few dense sink/tail slices of a pair
// (16 tokens each) are dealt round-robin to the warps that work on it.  Every warp streams its
// slices on its own:
//
//   * staging: each lane issues 16-byte cp.async copies of the slice's K nibbles (2 KB),
//     V codes (1 KB) and V scale/offset pairs (256 B) into a per-warp ring of three stages in
//     shared memory; a block's scales, role map and padding ride with its first slice;
//   * dequantisation never materialises K or V.  The descriptor-guided K decode is linear
//     in the stored nibbles, so once per block it is folded into the query:
//         score = sum_c w_c * nibble_c + const,
//     w_c = q_c s_c for a normal channel and 0 for the two slots of a salient channel; const
//     holds the -8 biases and the donors' padding values.  Nibbles are fed to the tensor
//     cores as fp16 SUBNORMALS: a nibble masked in place at bit 0 or 4 of a 16-bit lane is
//     the exact value nibble * 2^-24 (or * 2^-20), so unpacking costs one AND per two
//     elements and no integer-to-float conversion.  V works the same way with 2-bit codes
//     at bit 0..8 (ldmatrix.trans delivers token pairs per channel group), the per-token group
//     scale multiplied into the transposed probabilities and the group offsets contracted by
//     one more MMA;
//   * salient channels are rebuilt exactly as the reference rounds them: a tensor-core gather
//     (nibbles x selection matrix) yields 16*hi + lo, fl32((code - 128) * scale) is rounded to
//     the model dtype and contracted with the query at those channels;
//   * contractions use mma.sync.m16n8k16 with 16 tokens as M and the (up to 8) query heads
//     of the KV head as N, so one pass serves the whole GQA group; base-2 online softmax with
//     a lazily raised reference maximum.
#include <mutex>
#include <type_traits>

#include "common.cuh"
#include "exchange.cuh"

namespace inq {

constexpr int kWarps = 4;
constexpr int kThreads = kWarps * 32;
constexpr int kStages = 3;
// Tokens per loop iteration are a template parameter of the kernel: SUB = 2 (32 tokens) for
// blocks above 16 tokens, SUB = 1 (16 tokens) for smaller blocks (16-token pages), where every
// slice is a whole block and its metadata rides inside the slice's own ring stage.
// VK = 1: values stored as InQuant packed tensors like the keys (64 bytes of nibbles per token,
// per-channel scales per block, no per-token parameters).
// VK = 2: values as 4-bit codes with per-token scales and offsets for VG groups of 128 / VG channels.
template <int SUB, int VK = 0, int VG = 2>
struct SliceCfg {
  static constexpr int kSliceTokens = 16 * SUB;       // tokens staged and processed per loop iteration
  static constexpr int kStageK = 1024 * SUB, kStageV = (VK ? 1024 : 512) * SUB;
  static constexpr int kStageP = VK == 1 ? 0 : 16 * SUB * VG * 4;   // fp16 scale and offset per token and group
  static constexpr int kStageMeta = SUB == 1 ? 1024 : 0;   // K scales 512 B | role map 256 B | padding 256 B
  static constexpr int kStageBytes = kStageK + kStageV + kStageP + kStageMeta;
};
constexpr int kPlanSliceTokens = 32;                // the unit of the flat work list (equal for both SUB when a block has <= 16 tokens)
constexpr int kCtasPerSm = 3;                       // register budget: 168 per thread
constexpr int kRecordStride = 132;                  // floats per query head: acc[128], m, l, pad
constexpr int kRecordFloats = 8 * kRecordStride;    // one partial record (8 query heads)
constexpr int kQChunk = 36;                         // padded 32-float chunk of the staged query
constexpr int kQFragBytes = 8 * 32 * 8;              // the staged query as fp16 B fragments of the 8 K steps
constexpr int kQBytes = 8 * 4 * kQChunk * 4 + 64 + kQFragBytes;   // staged query, two factors per head, fragments
constexpr float kNegBig = -1.0e30f;
constexpr int kWarpFixed = 2048 + 256 + 64 + 64 + 2048 + 256;  // per-warp scratch before the per-group parts
constexpr float kRescaleSlack = 4.f;   // the running reference maximum may lag the true one by 2^4
// start value of a gather accumulator: -(128 + 128/512) in units of 2^-13, so that it ends as
// (code'_n - 128) + (code'_{n+8} - 128) / 512 (the fraction stays within +-1/4 even for a column
// whose second salient channel does not exist)
constexpr float kGatherInit = -128.25f / 8192.f;

// per-warp scratch of the InQuant-coded value side: staged block metadata (scales 512 B | role map
// 128 B | padding 64 B, padded to 768), per-lane flush tables (weight and constant of the lane's 16
// channels, their kinds) and the exchange area of the donor slots' sums
constexpr int kValueMeta = 768, kValueTables = 32 * (64 + 64 + 16), kValueXchg = 16 * 8 * 4;
constexpr int kValueScratch = 2 * kValueMeta + kValueTables + kValueXchg;   // two metadata slots, as for the keys
__host__ __device__ constexpr int warp_smem_bytes(int groups, int stage_bytes, int vk = 0) {
  return kWarpFixed + groups * (256 + 2048 + 64) + (vk ? kValueScratch : 0) + kStages * stage_bytes;
}

struct SeqDesc {
  const void* q;
  void* out;
  long long q_stride_h;
  const long long* table;        // table layout: [n_blocks][6] device pointers
  const signed char* roles;      // table layout: int8 [n_blocks][H][128]
  const unsigned char* pool;     // paged layout
  const int* page_table;         // paged layout: physical page of logical page i
  const void* sink_k; const void* sink_v; const void* tail_k; const void* tail_v;
  long long sink_k_sh, sink_k_st, sink_v_sh, sink_v_st;
  long long tail_k_sh, tail_k_st, tail_v_sh, tail_v_st;
  int n_blocks, sink_tokens, tail_tokens, first_visible, tail_skip;
  int pool_pages;
  const int* tail_tokens_dev;
  float* partial_out;            // optional: un-normalised (acc[128], m, l) per query head instead of `out`
  const void* new_k; const void* new_v;   // the step's new token (launches with fused_append)
  long long new_sh;
  int tail_capacity, reserved;
  const signed char* value_roles;   // table layout, InQuant-coded values: int8 [n_blocks][H][128]
};
static_assert(sizeof(SeqDesc) == sizeof(inq_decode_seq_t), "SeqDesc must mirror inq_decode_seq_t");

struct DecodeParams {
  const SeqDesc* seqs;
  SeqDesc one;
  int n_seq, H, G, T, n_pad;
  int n_ctas, n_pairs;
  long long per_cta, total_units, uniform_units;   // flat work decomposition (total_units counts the ramp units too)
  long long ramp_units;                            // list positions every pair is charged for its fixed costs
  const long long* pair_starts;                    // [n_pairs + 1] or nullptr when every pair has uniform_units
  float scale_log2e;
  long long page_bytes;
  int off_ks, off_km, off_kp, off_vp, off_vs, off_vo;
  float* partials;
  int* counters;
  int* status;
  int fused_append;
  const struct ExchangeView* exchange;   // device memory; set when the launch exchanges its records with the peer GPUs
};

// mirrors inq_decode_exchange_t
struct ExchangeView {
  unsigned char* inbox[kExMaxWorld];
  int* epoch;
  long long n_rows;
  int world, rank, spin_limit, reserved;
};
static_assert(sizeof(ExchangeView) == sizeof(inq_decode_exchange_t), "ExchangeView must mirror inq_decode_exchange_t");

struct BlockPtrs {
  const unsigned char *kp, *ks, *kr, *kpad, *vp, *vs, *vo, *vr;
};

// ------------------------------------------------------------------------------------------ PTX helpers
__device__ __forceinline__ void mma_f16(float (&d)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0,
                                        unsigned b1) {
  asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3},{%4,%5,%6,%7},{%8,%9},{%0,%1,%2,%3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0,
                                         unsigned b1) {
  asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3},{%4,%5,%6,%7},{%8,%9},{%0,%1,%2,%3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
template <typename QT>
__device__ __forceinline__ void mma_qt(float (&d)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0,
                                       unsigned b1) {
  if (sizeof(QT) == 2 && std::is_same<QT, __half>::value)
    mma_f16(d, a0, a1, a2, a3, b0, b1);
  else
    mma_bf16(d, a0, a1, a2, a3, b0, b1);
}
__device__ __forceinline__ unsigned movmatrix_trans(unsigned x) {
  unsigned y;
  asm("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(y) : "r"(x));
  return y;
}
__device__ __forceinline__ void cp_async16(void* dst, const void* src) {
  unsigned d = (unsigned)__cvta_generic_to_shared(dst);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(src));
}
__device__ __forceinline__ void cp_async4(void* dst, const void* src) {
  unsigned d = (unsigned)__cvta_generic_to_shared(dst);
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(d), "l"(src));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N));
}
// Shared-memory loads through 32-bit shared addresses with compile-time byte offsets.  They are
// pure asm statements so that the compiler may schedule them freely among the MMAs; an address
// passed through launder() after a synchronisation point cannot be read before that point, nor
// can its loads be merged with those of an earlier loop iteration.
__device__ __forceinline__ unsigned launder(unsigned addr) {
  asm volatile("" : "+r"(addr));
  return addr;
}
template <int OFF>
__device__ __forceinline__ uint4 lds128(unsigned addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4+%5];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr), "n"(OFF));
  return v;
}
template <int OFF>
__device__ __forceinline__ uint2 lds64(unsigned addr) {
  uint2 v;
  asm volatile("ld.shared.v2.u32 {%0,%1}, [%2+%3];" : "=r"(v.x), "=r"(v.y) : "r"(addr), "n"(OFF));
  return v;
}
template <int OFF>
__device__ __forceinline__ unsigned lds32(unsigned addr) {
  unsigned v;
  asm volatile("ld.shared.u32 %0, [%1+%2];" : "=r"(v) : "r"(addr), "n"(OFF));
  return v;
}
// four transposed 8x8 b16 matrices: register i of lane (r, j) holds elements (2j, r) and (2j+1, r) of matrix i
template <int OFF>
__device__ __forceinline__ uint4 ldsm4_trans(unsigned addr) {
  uint4 v;
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4+%5];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr), "n"(OFF));
  return v;
}
__device__ __forceinline__ unsigned hmul2_bits(unsigned a, unsigned b) {
  unsigned d;
  asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}
__device__ __forceinline__ unsigned smem_addr(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
// D = A*B with a zero accumulator (first step of a chain: nothing to keep live or to clear)
__device__ __forceinline__ void mma_f16_first(float (&d)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0,
                                              unsigned b1) {
  asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3},{%4,%5,%6,%7},{%8,%9},{%10,%10,%10,%10};"
               : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.f));
}
// D = A*B + c with the same constant c in all four accumulators (first step of a chain)
__device__ __forceinline__ void mma_f16_init(float (&d)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0,
                                             unsigned b1, float c) {
  asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3},{%4,%5,%6,%7},{%8,%9},{%10,%10,%10,%10};"
               : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(c));
}
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ unsigned pack_half2(float lo, float hi) {
  __half2 h = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<unsigned*>(&h);
}
template <typename QT>
__device__ __forceinline__ unsigned pack_qt2(float lo, float hi) {
  if (std::is_same<QT, __half>::value) return pack_half2(lo, hi);
  __nv_bfloat162 b = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<unsigned*>(&b);
}
__device__ __forceinline__ float2 half2_bits_to_float2(unsigned bits) {
  return __half22float2(*reinterpret_cast<__half2*>(&bits));
}

// ------------------------------------------------------------------------------------------ block lookup
template <int MODE, int VK = 0, int VG = 2>
__device__ __forceinline__ BlockPtrs locate_block(const DecodeParams& P, const long long* table,
                                                  const signed char* roles, const unsigned char* pool,
                                                  const int* page_table, int pool_pages, int b, int h,
                                                  const signed char* value_roles = nullptr) {
  BlockPtrs out;
  out.vr = nullptr;
  if (MODE == 0) {
    const long long* row = table + (long long)b * 6;
    const long long T = P.T;
    out.kp = (const unsigned char*)row[0] + (long long)h * T * 64;
    out.ks = (const unsigned char*)row[1] + (long long)h * 512;
    out.kpad = (const unsigned char*)row[2] + (long long)h * P.n_pad * 4;
    if (VK == 1) {
      // values coded like the keys: payload, per-channel scales, padding list, role map
      out.vp = (const unsigned char*)row[3] + (long long)h * T * 64;
      out.vs = (const unsigned char*)row[4] + (long long)h * 512;
      out.vo = (const unsigned char*)row[5] + (long long)h * 64;
      out.vr = (const unsigned char*)value_roles + ((long long)b * P.H + h) * 128;
    } else if (VK == 2) {
      out.vp = (const unsigned char*)row[3] + (long long)h * T * 64;
      out.vs = (const unsigned char*)row[4] + (long long)h * T * (2 * VG);
      out.vo = (const unsigned char*)row[5] + (long long)h * T * (2 * VG);
    } else {
      out.vp = (const unsigned char*)row[3] + (long long)h * T * 32;
      out.vs = (const unsigned char*)row[4] + (long long)h * T * (2 * VG);
      out.vo = (const unsigned char*)row[5] + (long long)h * T * (2 * VG);
    }
    out.kr = (const unsigned char*)roles + ((long long)b * P.H + h) * 128;
  } else {
    int id = page_table[b];
    if (pool_pages > 0 && (unsigned)id >= (unsigned)pool_pages) {
      // never dereferenced: the first page stands in and the caller learns of it from the status word
      atomicOr(P.status, INQ_STATUS_BAD_INDEX);
      id = 0;
    }
    const unsigned char* page = pool + (long long)id * P.page_bytes;
    const long long T = P.T;
    out.kp = page + (long long)h * T * 64;
    out.ks = page + P.off_ks + (long long)h * 512;
    out.kr = page + P.off_km + (long long)h * 256;
    out.kpad = page + P.off_kp + (long long)h * 64;
    out.vp = page + P.off_vp + (long long)h * T * 32;
    out.vs = page + P.off_vs + (long long)h * T * 4;
    out.vo = page + P.off_vo + (long long)h * T * 4;
  }
  return out;
}

// Issue the asynchronous copies of one packed slice (32 tokens from `tok0`) into a stage.
// Stage layout: K nibbles [32 tokens][64 B]; V codes [32 tokens][2 x 16 B] with the two halves
// of tokens 4..7 (mod 8) swapped so that the later word reads of tokens 2j, 2j+1, 2j+8, 2j+9
// fall into distinct banks; V scale pairs [32] and V offset pairs [32] (4 B each).
template <int kSub>
__device__ __forceinline__ void stage_slice(unsigned char* stage, const unsigned char* kp, const unsigned char* vp,
                                            const unsigned char* vs, const unsigned char* vo, int tok0, int T, int lane) {
  constexpr int kSliceTokens = SliceCfg<kSub>::kSliceTokens;
  constexpr int kStageK = SliceCfg<kSub>::kStageK, kStageV = SliceCfg<kSub>::kStageV, kStageP = SliceCfg<kSub>::kStageP;
  const int v_dst = kStageK + (((lane >> 1) * 2 + ((lane & 1) ^ ((lane >> 3) & 1))) << 4);
  // parameter vectors: 4 bytes (two fp16 group values) per token; with 16-token slices the lower
  // half-warp copies the scales and the upper half-warp the offsets
  const int p_tok = kSub == 1 ? (lane & 15) : lane;
  const bool p_both = kSub > 1;
  if (tok0 + kSliceTokens <= T) {
    // every token exists: K tile, V tile and parameter vectors are contiguous in global memory
    const unsigned char* ksrc = kp + tok0 * 64 + lane * 16;
#pragma unroll
    for (int k = 0; k < 2 * kSub; ++k) cp_async16(stage + lane * 16 + k * 512, ksrc + k * 512);
    const unsigned char* vsrc = vp + tok0 * 32 + lane * 16;
#pragma unroll
    for (int k = 0; k < kSub; ++k) cp_async16(stage + v_dst + k * 512, vsrc + k * 512);
    if (p_both) {
      cp_async4(stage + kStageK + kStageV + lane * 4, vs + (tok0 + lane) * 4);
      cp_async4(stage + kStageK + kStageV + kStageP / 2 + lane * 4, vo + (tok0 + lane) * 4);
    } else {
      cp_async4(stage + kStageK + kStageV + (lane < 16 ? 0 : kStageP / 2) + p_tok * 4, (lane < 16 ? vs : vo) + (tok0 + p_tok) * 4);
    }
  } else {
    const int last = T - 1;
    const int r = lane >> 2, j = lane & 3;
#pragma unroll
    for (int k = 0; k < 2 * kSub; ++k)
      cp_async16(stage + lane * 16 + k * 512, kp + min(tok0 + r + 8 * k, last) * 64 + j * 16);
#pragma unroll
    for (int k = 0; k < kSub; ++k)
      cp_async16(stage + v_dst + k * 512, vp + min(tok0 + (lane >> 1) + 16 * k, last) * 32 + (lane & 1) * 16);
    const int tp = min(tok0 + p_tok, last);
    if (p_both) {
      cp_async4(stage + kStageK + kStageV + lane * 4, vs + tp * 4);
      cp_async4(stage + kStageK + kStageV + kStageP / 2 + lane * 4, vo + tp * 4);
    } else {
      cp_async4(stage + kStageK + kStageV + (lane < 16 ? 0 : kStageP / 2) + p_tok * 4, (lane < 16 ? vs : vo) + tp * 4);
    }
  }
}

// ------------------------------------------------------------------------------------------ exchange of a pair
// Split-KV across GPUs, run by the CTA that has just merged this rank's parts of a pair: the
// pair's un-normalised record (eight channels per thread in `oa`, `ob`; `top`, `l` of the row) goes
// into every peer's inbox over NVLink peer memory, the peers' records of the same pair are awaited
// in this rank's own inbox and all records are merged in rank order, so every rank writes
// bit-identical output rows.
// Every 32-bit word of a record travels as ONE 8-byte store {word, step number}: such a store is
// indivisible, so a word whose tag equals the current step is the word of this step and neither a
// fence nor a separate flag is needed (a system-scope fence inside this kernel was measured at 9 us:
// it queues behind the copies the other CTAs of the SM still have in flight).  A reader polls the
// words it needs until their tags match -- bounded: a wait that runs out raises
// INQ_STATUS_WAIT_TIMEOUT and zeroes the rows.  The inbox is double buffered by step parity.
// All threads of the CTA call it; those with g < g_valid hold a row.  The step number comes from
// the epoch word that the launch advances when its last CTA leaves.
__device__ __forceinline__ void st_tagged(uint2* p, unsigned word, unsigned tag) {
  asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(p), "r"(word), "r"(tag) : "memory");
}
__device__ __forceinline__ uint4 ld_tagged2(const uint2* p) {   // two tagged words
  uint4 v;
  asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}
template <typename QT>
__device__ __noinline__ void exchange_pair(const ExchangeView* X, int pair, long long row0, int g, int g_valid, int c8,
                                           float4 oa, float4 ob, float top, float l, QT* out, int* status,
                                           float* scratch) {
  __shared__ int s_failed;
  const int tid = threadIdx.x;
  const bool active = g < g_valid;
  const long long row = row0 + g;
  const int world = X->world, me = X->rank;
  const long long n_rows = X->n_rows;
  const unsigned step = (unsigned)(X->epoch[0] + 1);
  const int parity = (int)(step & 1u);
  unsigned char* const own = X->inbox[me];
  if (tid == 0) s_failed = 0;
  // the pair's rows are adjacent in an inbox: staged in shared memory, they leave as consecutive
  // 8-byte stores of consecutive threads (whole 128-byte lines over NVLink, not scattered sectors)
  if (active) {
    float* const rec = scratch + g * kExRowFloats;
    *(float2*)(rec + c8) = make_float2(oa.x, oa.y);
    *(float2*)(rec + c8 + 2) = make_float2(oa.z, oa.w);
    *(float2*)(rec + c8 + 4) = make_float2(ob.x, ob.y);
    *(float2*)(rec + c8 + 6) = make_float2(ob.z, ob.w);
    if (c8 == 0) *(float2*)(rec + 128) = make_float2(top, l);
  }
  __syncthreads();
  {
    const int n_words = g_valid * kExRowFloats;
    const unsigned* const src = (const unsigned*)scratch;
    // every rank starts with the peer after itself, so that no inbox is everybody's first target
    for (int hop = 1; hop < world; ++hop) {
      const int p = me + hop < world ? me + hop : me + hop - world;
      uint2* const dst = ex_tagged(X->inbox[p], parity, me, world, n_rows) + row0 * kExRowFloats;
      for (int i = tid; i < n_words; i += kThreads) st_tagged(dst + i, src[i], step);
    }
  }
  (void)pair;
  // this thread's words of every peer's record (channels c8 .. c8+7 and (m, l) of its row) are awaited
  // first; only (m, l) are kept, the channels are read again when the records are summed in rank order
  float peer_m[kExMaxWorld], peer_l[kExMaxWorld];
  bool failed_here = false;
  if (active) {
    const int limit = X->spin_limit > 0 ? X->spin_limit : kExDefaultSpin;
#pragma unroll
    for (int p = 0; p < kExMaxWorld; ++p) {
      peer_m[p] = 0.f;
      peer_l[p] = 0.f;
      if (p >= world || p == me || failed_here) continue;
      const uint2* const rec = ex_tagged(own, parity, p, world, n_rows) + row * kExRowFloats;
      int polls = 0;
      while (true) {
        const uint4 w0 = ld_tagged2(rec + c8), w1 = ld_tagged2(rec + c8 + 2), w2 = ld_tagged2(rec + c8 + 4);
        const uint4 w3 = ld_tagged2(rec + c8 + 6), w4 = ld_tagged2(rec + 128);
        const bool here = w0.y == step && w0.w == step && w1.y == step && w1.w == step && w2.y == step && w2.w == step &&
                          w3.y == step && w3.w == step && w4.y == step && w4.w == step;
        if (here) {
          peer_m[p] = __uint_as_float(w4.x);
          peer_l[p] = __uint_as_float(w4.z);
          break;
        }
        if (++polls > limit) {
          failed_here = true;
          break;
        }
        __nanosleep(40);
      }
    }
    if (failed_here) atomicOr(&s_failed, 1);
  }
  __syncthreads();
  const bool failed = s_failed != 0;
  if (failed && tid == 0) atomicOr(status, INQ_STATUS_WAIT_TIMEOUT);
  if (active) {
    float o[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f}, norm = 1.f;
    if (!failed) {
      float all_top = top;
#pragma unroll
      for (int p = 0; p < kExMaxWorld; ++p)
        if (p < world && p != me) all_top = fmaxf(all_top, peer_m[p]);
      norm = 0.f;
#pragma unroll
      for (int p = 0; p < kExMaxWorld; ++p) {
        if (p >= world) continue;
        if (p == me) {
          const float w = fast_exp2(top - all_top);
          norm = fmaf(l, w, norm);
          o[0] = fmaf(oa.x, w, o[0]); o[1] = fmaf(oa.y, w, o[1]); o[2] = fmaf(oa.z, w, o[2]); o[3] = fmaf(oa.w, w, o[3]);
          o[4] = fmaf(ob.x, w, o[4]); o[5] = fmaf(ob.y, w, o[5]); o[6] = fmaf(ob.z, w, o[6]); o[7] = fmaf(ob.w, w, o[7]);
        } else {
          const uint2* const rec = ex_tagged(own, parity, p, world, n_rows) + row * kExRowFloats + c8;
          const uint4 w0 = ld_tagged2(rec), w1 = ld_tagged2(rec + 2), w2 = ld_tagged2(rec + 4), w3 = ld_tagged2(rec + 6);
          const float w = fast_exp2(peer_m[p] - all_top);
          norm = fmaf(peer_l[p], w, norm);
          o[0] = fmaf(__uint_as_float(w0.x), w, o[0]); o[1] = fmaf(__uint_as_float(w0.z), w, o[1]);
          o[2] = fmaf(__uint_as_float(w1.x), w, o[2]); o[3] = fmaf(__uint_as_float(w1.z), w, o[3]);
          o[4] = fmaf(__uint_as_float(w2.x), w, o[4]); o[5] = fmaf(__uint_as_float(w2.z), w, o[5]);
          o[6] = fmaf(__uint_as_float(w3.x), w, o[6]); o[7] = fmaf(__uint_as_float(w3.z), w, o[7]);
        }
      }
    }
#pragma unroll
    for (int k = 0; k < 8; ++k) out[k] = from_float<QT>(failed ? 0.f : o[k] / norm);
  }
}

// ------------------------------------------------------------------------------------------ the kernel
// FAST: blocks of whole 32-token slices, at least two per block, exactly one group of 16 salient
// channels (the preset and the 128/256-token pages): the copies of a slice then are eight
// asynchronous copies from per-lane pointers that advance by constants, a block's metadata is
// requested as soon as the prefetch cursor enters the block, and nothing ragged is handled.
// VK = 1 (with FAST, table layout): the values are InQuant packed tensors like the keys.  Their
// nibbles go through the value MMAs as fp16 subnormals into accumulators of the current block
// alone; when the block ends these are folded into the running output with the block's
// per-channel scales (regular channel: s (sum p code - 8 sum p); salient: s (16 sum p hi + sum p lo
// - 128 sum p), the low-nibble sum fetched from the lane that owns the donor slot; donor: its
// constant times sum p).  The second accumulator set needs the registers of two CTAs per SM.
// VK = 2 (same geometry): 4-bit values with per-token scales and offsets for VG = 4, 2 or 1 groups
// of 32, 64 or 128 channels.  The nibbles take the value MMAs of the coded values, the group scale is
// multiplied into the probabilities and the offsets are contracted by one more MMA as for the 2-bit
// values; a 16-byte chunk of a value row (8 words of four nibbles) is 32 channels, so every MMA lies
// inside one group.  Their stages are 4.1 to 4.5 KB, so two CTAs fit an SM here as well.
template <int MODE, typename QT, bool SAL, int SUB, bool FAST, int VK = 0, int VG = 2>
__global__ void __launch_bounds__(kThreads, VK ? 2 : kCtasPerSm) decode_kernel(const DecodeParams P) {
  static_assert(!VK || (FAST && MODE == 0 && SAL && SUB == 2), "coded and 4-bit values: whole-slice path of the table layout only");
  static_assert(VK == 2 ? (VG == 1 || VG == 2 || VG == 4) : VK == 0 ? (VG == 2 || ((VG == 1 || VG == 4) && FAST && MODE == 0)) : VG == 2,
                "4-bit values: groups of 32, 64 or 128 channels; 2-bit values: 64, or 32 and 128 on the whole-slice path");
  constexpr int kSub = SUB;
  constexpr int kSliceTokens = SliceCfg<SUB, VK, VG>::kSliceTokens;
  constexpr int kStageK = SliceCfg<SUB, VK, VG>::kStageK, kStageV = SliceCfg<SUB, VK, VG>::kStageV, kStageP = SliceCfg<SUB, VK, VG>::kStageP;
  constexpr int kStageBytes = SliceCfg<SUB, VK, VG>::kStageBytes;
  constexpr bool kMetaInStage = SliceCfg<SUB, VK, VG>::kStageMeta > 0;   // host guarantees one slice per block
  constexpr int kMetaOffset = kStageK + kStageV + kStageP;
  extern __shared__ __align__(16) unsigned char smem[];
  float* qs = (float*)smem;                                             // 8 heads x 4 chunks x kQChunk
  float* qinv = qs + 8 * 4 * kQChunk;   // per head: softmax scale * log2(e) * 2^(exponent of max|q| - 12)
  float* qunscale = qinv + 8;           // per head: the power of two that restores the staged query
  // the staged query once more as fp16 pairs in B-fragment order: entry [K step][lane (head r, chunk j)]
  // holds channels (c, c+4 | c+1, c+5), c = 32j + 8 (step / 2) + 2 (step % 2), of query head r
  unsigned char* qfrag = (unsigned char*)(qunscale + 8);
  unsigned char* warp_base = smem + kQBytes;
  const int warp = __shfl_sync(0xffffffffu, (int)(threadIdx.x >> 5), 0), lane = threadIdx.x & 31;
  const int r = lane >> 2, j = lane & 3;
  const int n_pad = FAST ? 16 : P.n_pad;                                // salient channels per head
  const int groups = FAST ? 1 : (n_pad + 15) >> 4;                      // ... in groups of 16
  const int warp_bytes = warp_smem_bytes(groups, kStageBytes, VK == 1);
  unsigned char* const wb = warp_base + warp * warp_bytes;
  // folded-query B fragments of the 8 K steps ([step][lane] x 8 bytes); while a block's weights
  // are being derived the same 2 KB hold the per-channel slot weights and additive constants
  unsigned char* wW = wb;
  float* wssc = (float*)(wb + 2048);                                    // scale of salient channel i
  unsigned char* wsrc = (unsigned char*)(wssc + 64);                    // channel of salient i
  unsigned char* wdon = wsrc + 64;                                      // its donor slot
  // staged block metadata: K scales 512 B | role map 256 B | padding 256 B.  Two slots: the whole-slice
  // path stages block b into slot b % 2, so the block after the one being consumed can be requested
  // while this one's slot is still to be read
  unsigned char* wmeta = wdon + 64;
  unsigned char* wfrag = wmeta + 2048;    // a block's channel weights as fp16 pairs in B-fragment order: [K step][chunk] x 8 B
  unsigned char* wqsal = wb + kWarpFixed;                               // B fragments: query at salient channels
  unsigned char* wsel = wqsal + groups * 256;                           // B fragments: nibble selection
  unsigned short* wcell = (unsigned short*)(wsel + groups * 2048);      // selection cells written by the last fold (offsets into wsel)
  // InQuant-coded values: staged value metadata of a block, the lane's flush tables, the donor sums
  unsigned char* wvmeta = (unsigned char*)wcell + groups * 64;
  float* wvw = (float*)(wvmeta + 2 * kValueMeta);                       // [lane][16] weight of the block sum
  float* wvk = wvw + 32 * 16;                                           // [lane][16] factor of sum p
  signed char* wvkind = (signed char*)(wvk + 32 * 16);                  // [lane][16] -1 regular, idx salient, 16 + idx donor
  float* wvx = (float*)(wvkind + 32 * 16);                              // [16 list entries][8 heads] low-nibble sums
  unsigned char* ring = (unsigned char*)wcell + groups * 64 + (VK == 1 ? kValueScratch : 0);
  __shared__ int s_is_last;

  // Flat decomposition: the packed slices of all (sequence, KV head, head tile) pairs form one
  // list that is cut into gridDim.x equal ranges; a CTA walks its range pair by pair.
  const int gtiles = (P.G + 7) >> 3;
  // Every pair starts with `ramp_units` list positions that hold no slices: they stand for the
  // fixed cost a CTA pays per pair it touches (query staging, first copies, dense slices, record,
  // merge), so a CTA whose range crosses into the next pair is given fewer slices.  A CTA that
  // reaches only the ramp of a pair leaves that pair alone.
  const long long R = P.ramp_units;
  const long long c_begin = (long long)blockIdx.x * P.per_cta;
  const long long c_end = min(c_begin + P.per_cta, P.total_units);
  long long pos = c_begin;
  int pair;
  if (P.pair_starts) {
    int lo = 0, hi = P.n_pairs - 1;
    while (lo < hi) {
      const int mid = (lo + hi + 1) >> 1;
      if (P.pair_starts[mid] + mid * R <= pos) lo = mid; else hi = mid - 1;
    }
    pair = lo;
  } else {
    pair = (int)(pos / (P.uniform_units + R));
  }
  for (; pos < c_end; ++pair) {
  const long long pair_lo = (P.pair_starts ? P.pair_starts[pair] : (long long)pair * P.uniform_units) + (pair + 1) * R;   // first slice
  const long long pair_hi = (P.pair_starts ? P.pair_starts[pair + 1] : (long long)(pair + 1) * P.uniform_units) + (pair + 1) * R;
  const long long seg_lo = max(pos, pair_lo) - pair_lo, seg_hi = min(c_end, pair_hi) - pair_lo;
  pos = min(c_end, pair_hi);
  if (seg_hi <= seg_lo) continue;   // only ramp positions of this pair fall into the range
  const int first_cta = (int)(pair_lo / P.per_cta), last_cta = (int)((pair_hi - 1) / P.per_cta);
  const int n_cta_pair = last_cta - first_cta + 1;
  const int seq = pair / (P.H * gtiles);
  const int h = (pair / gtiles) % P.H, gt = pair % gtiles;
  // Descriptor fields are fetched where they are used: from kernel parameters for a single
  // sequence, from the device array for a batch.
  const SeqDesc* const Dp = P.seqs ? P.seqs + seq : nullptr;
#define SEQ(field) (Dp ? Dp->field : P.one.field)
  const long long* const d_table = SEQ(table);
  const signed char* const d_roles = SEQ(roles);
  const unsigned char* const d_pool = SEQ(pool);
  const int* const d_pages = SEQ(page_table);
  const int d_pool_pages = SEQ(pool_pages);
  // coded values without their role map: never dereferenced, the key map stands in and the caller
  // learns of it from the status word
  const signed char* d_vroles = VK == 1 ? SEQ(value_roles) : nullptr;
  if (VK == 1 && d_vroles == nullptr) {
    if (threadIdx.x == 0) atomicOr(P.status, INQ_STATUS_BAD_INDEX);
    d_vroles = d_roles;
  }
  const int first_visible = SEQ(first_visible);
  // (loaded here, ahead of the barriers of the query staging, so that their latency overlaps it)
  const int T = P.T;
  const int spb = (T + kSliceTokens - 1) / kSliceTokens;   // packed slices per block
  const int n_blocks = SEQ(n_blocks);
  const int sink_tokens = SEQ(sink_tokens);
  const int* const tail_dev = SEQ(tail_tokens_dev);
  const int tail_tokens = tail_dev ? *tail_dev : SEQ(tail_tokens);
  const int g_valid = min(8, P.G - gt * 8);
  const long long q_head0 = (long long)h * P.G + gt * 8;
  const QT* qptr = (const QT*)SEQ(q);
  const long long q_stride = SEQ(q_stride_h);

  // the merge of the previous pair may have used this scratch: start from an empty selection
  // matrix and an empty list of written cells
  for (int v = lane; v < groups * 128; v += 32) ((uint4*)wsel)[v] = make_uint4(0u, 0u, 0u, 0u);
  for (int v = lane; v < 64; v += 32) wssc[v] = 0.f;   // scales of unused salient slots must be finite
  for (int v = lane; v < groups * 32; v += 32) wcell[v] = 0;
  // query as fp32, chunked so that lanes (head, chunk) read distinct banks, then scaled per head by
  // a power of two that brings its largest magnitude into [2^12, 2^13): every folded weight is
  // then a product below 2^14 that fp16 holds without overflow and with full precision
  if ((((unsigned long long)qptr | (unsigned long long)(q_stride * (long long)sizeof(QT))) & 15ull) == 0) {
    // one 16-byte load per thread: head g = thread / 16, channels 8 * (thread % 16) .. + 7
    const int g = threadIdx.x >> 4, c0 = (threadIdx.x & 15) * 8;
    uint4 raw = make_uint4(0u, 0u, 0u, 0u);
    if (g < g_valid) raw = *(const uint4*)(qptr + (q_head0 + g) * q_stride + c0);
    const QT* e = (const QT*)&raw;
    float* dst = qs + (g * 4 + (c0 >> 5)) * kQChunk + (c0 & 31);
    *(float4*)dst = make_float4(to_float<QT>(e[0]), to_float<QT>(e[1]), to_float<QT>(e[2]), to_float<QT>(e[3]));
    *(float4*)(dst + 4) = make_float4(to_float<QT>(e[4]), to_float<QT>(e[5]), to_float<QT>(e[6]), to_float<QT>(e[7]));
  } else {
    for (int idx = threadIdx.x; idx < 8 * 128; idx += kThreads) {
      int g = idx >> 7, c = idx & 127;
      float v = g < g_valid ? to_float<QT>(qptr[(q_head0 + g) * q_stride + c]) : 0.f;
      qs[(g * 4 + (c >> 5)) * kQChunk + (c & 31)] = v;
    }
  }
  __syncthreads();
#pragma unroll
  for (int hh = 0; hh < 8 / kWarps; ++hh) {
    const int head = warp * (8 / kWarps) + hh;
    float* row = qs + head * 4 * kQChunk + lane;
    const float v0 = row[0], v1 = row[kQChunk], v2 = row[2 * kQChunk], v3 = row[3 * kQChunk];
    unsigned top = __float_as_uint(fmaxf(fmaxf(fabsf(v0), fabsf(v1)), fmaxf(fabsf(v2), fabsf(v3))));
    top = __reduce_max_sync(0xffffffffu, top);
    int ex = (int)(top >> 23) - 127;
    ex = top == 0u ? 0 : max(-60, min(60, ex));
    const float mul = __uint_as_float((unsigned)(127 + 12 - ex) << 23);
    row[0] = v0 * mul; row[kQChunk] = v1 * mul; row[2 * kQChunk] = v2 * mul; row[3 * kQChunk] = v3 * mul;
    if (lane == 0) {
      qunscale[head] = __uint_as_float((unsigned)(127 + ex - 12) << 23);
      qinv[head] = P.scale_log2e * qunscale[head];
    }
  }
  __syncthreads();
  for (int e = threadIdx.x; e < 8 * 32; e += kThreads) {
    const int ks = e >> 5, fr = (e & 31) >> 2, fj = e & 3;
    const float* src = qs + (fr * 4 + fj) * kQChunk + 8 * (ks >> 1) + 2 * (ks & 1);
    *(uint2*)(qfrag + e * 8) = make_uint2(pack_half2(src[0], src[4]), pack_half2(src[1], src[5]));
  }
  __syncthreads();
  const long long n_packed = (long long)n_blocks * spb;
  const int sink_slices = (sink_tokens + 15) >> 4, tail_slices = (tail_tokens + 15) >> 4;
  // packed slices are cut evenly over all warps of this (sequence, KV head); the few dense
  // slices are dealt round-robin so that no warp ends with a long exposed-latency tail
  const int n_workers = n_cta_pair * kWarps, worker = ((int)blockIdx.x - first_cta) * kWarps + warp;
  const long long pa = min(n_packed, seg_lo + (seg_hi - seg_lo) * warp / kWarps);
  const long long pb = min(n_packed, seg_lo + (seg_hi - seg_lo) * (warp + 1) / kWarps);
  // with a fused append the step's new token is one more dense slice: it is read from the caller's
  // rows (tail_tokens counts the tokens before it) and stored behind the tail for the next steps
  const bool has_new = P.fused_append && SEQ(new_k) != nullptr;
  const int n_dense = sink_slices + tail_slices + (has_new ? 1 : 0);

  float m_run[2] = {kNegBig, kNegBig}, l_run[2] = {0.f, 0.f};
  float acc[8][4];
#pragma unroll
  for (int mt = 0; mt < 8; ++mt)
#pragma unroll
    for (int k = 0; k < 4; ++k) acc[mt][k] = 0.f;
  float oacc[4] = {0.f, 0.f, 0.f, 0.f};   // value offsets: row = value group (lanes r < 2), columns = heads 2j, 2j+1

  // ---------------------------------------------------------------- exact sink and tail
  // (run while the first packed slices are still in flight, see below)
  auto dense_part = [&]() {
  if (worker < n_dense) {
    unsigned qf[16];
    {
      const bool live = r < g_valid;
#pragma unroll
      for (int m = 0; m < 4; ++m) {
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (live) v = *(const uint4*)(qptr + (q_head0 + r) * q_stride + (4 * m + j) * 8);
        qf[4 * m + 0] = v.x; qf[4 * m + 1] = v.y; qf[4 * m + 2] = v.z; qf[4 * m + 3] = v.w;
      }
    }
    for (int ds = worker; ds < n_dense; ds += n_workers) {
      const bool is_sink = ds < sink_slices;
      const bool is_new = ds >= sink_slices + tail_slices;   // the step's new token: a slice of one row
      const int tok0 = is_new ? 0 : (is_sink ? ds : ds - sink_slices) * 16;
      const int count = is_new ? 1 : is_sink ? sink_tokens : tail_tokens;
      const int skip = is_sink || is_new ? 0 : SEQ(tail_skip);
      const QT* kb = is_new ? (const QT*)SEQ(new_k) + (long long)h * SEQ(new_sh)
                            : (const QT*)(is_sink ? SEQ(sink_k) : SEQ(tail_k)) + (long long)h * (is_sink ? SEQ(sink_k_sh) : SEQ(tail_k_sh));
      const QT* vb = is_new ? (const QT*)SEQ(new_v) + (long long)h * SEQ(new_sh)
                            : (const QT*)(is_sink ? SEQ(sink_v) : SEQ(tail_v)) + (long long)h * (is_sink ? SEQ(sink_v_sh) : SEQ(tail_v_sh));
      const long long kst = is_new ? 0 : is_sink ? SEQ(sink_k_st) : SEQ(tail_k_st), vst = is_new ? 0 : is_sink ? SEQ(sink_v_st) : SEQ(tail_v_st);
      if (is_new && gt == 0) {
        // one warp per (sequence, KV head) stores the token behind the tail; this launch reads it
        // from the caller's rows only, so the store races with nothing
        if (tail_tokens < SEQ(tail_capacity)) {
          QT* dst = (QT*)(lane < 16 ? SEQ(tail_k) : SEQ(tail_v)) + (long long)h * (lane < 16 ? SEQ(tail_k_sh) : SEQ(tail_v_sh)) +
                    (long long)tail_tokens * (lane < 16 ? SEQ(tail_k_st) : SEQ(tail_v_st));
          *((uint4*)dst + (lane & 15)) = *((const uint4*)(lane < 16 ? kb : vb) + (lane & 15));
        } else if (lane == 0) {
          atomicOr(P.status, INQ_STATUS_BAD_INDEX);
        }
      }
      const int last = count - 1;
      float S[4] = {0.f, 0.f, 0.f, 0.f};
      // the value rows are requested together with the key rows: one exposed latency, not two
      const QT* vA = vb + (long long)min(tok0 + 2 * j, last) * vst;
      const QT* vB = vb + (long long)min(tok0 + 2 * j + 1, last) * vst;
      const QT* vC = vb + (long long)min(tok0 + 2 * j + 8, last) * vst;
      const QT* vD = vb + (long long)min(tok0 + 2 * j + 9, last) * vst;
      uint4 vrow[2][4];
      uint2 vrow2[4][4];   // coded values: this lane's channels are 32 wg + 4 r .. + 3 (see the value MMAs below)
      {
        const QT* k_lo = kb + (long long)min(tok0 + r, last) * kst;
        const QT* k_hi = kb + (long long)min(tok0 + r + 8, last) * kst;
        uint4 x[4], y[4];
#pragma unroll
        for (int m = 0; m < 4; ++m) {
          x[m] = *(const uint4*)(k_lo + (4 * m + j) * 8);
          y[m] = *(const uint4*)(k_hi + (4 * m + j) * 8);
        }
        if (VK) {
#pragma unroll
          for (int wg = 0; wg < 4; ++wg) {
            const int ch = 32 * wg + 4 * r;
            vrow2[wg][0] = *(const uint2*)(vA + ch);
            vrow2[wg][1] = *(const uint2*)(vB + ch);
            vrow2[wg][2] = *(const uint2*)(vC + ch);
            vrow2[wg][3] = *(const uint2*)(vD + ch);
          }
        } else {
#pragma unroll
          for (int gr = 0; gr < 2; ++gr) {
            const int ch = 64 * gr + 8 * r;
            vrow[gr][0] = *(const uint4*)(vA + ch);
            vrow[gr][1] = *(const uint4*)(vB + ch);
            vrow[gr][2] = *(const uint4*)(vC + ch);
            vrow[gr][3] = *(const uint4*)(vD + ch);
          }
        }
#pragma unroll
        for (int m = 0; m < 4; ++m) {
          mma_qt<QT>(S, x[m].x, y[m].x, x[m].y, y[m].y, qf[4 * m + 0], qf[4 * m + 1]);
          mma_qt<QT>(S, x[m].z, y[m].z, x[m].w, y[m].w, qf[4 * m + 2], qf[4 * m + 3]);
        }
      }
      float s2[4] = {S[0] * P.scale_log2e, S[1] * P.scale_log2e, S[2] * P.scale_log2e, S[3] * P.scale_log2e};
      {
        const bool lo_ok = tok0 + r < count && tok0 + r >= skip;
        const bool hi_ok = tok0 + r + 8 < count && tok0 + r + 8 >= skip;
        if (!lo_ok) s2[0] = s2[1] = -INFINITY;
        if (!hi_ok) s2[2] = s2[3] = -INFINITY;
      }
      float mx0 = fmaxf(s2[0], s2[2]), mx1 = fmaxf(s2[1], s2[3]);
#pragma unroll
      for (int off = 4; off < 32; off <<= 1) {
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, off));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, off));
      }
      const float mn0 = fmaxf(m_run[0], mx0), mn1 = fmaxf(m_run[1], mx1);
      if (__any_sync(0xffffffffu, mn0 > m_run[0] || mn1 > m_run[1])) {
        const float a0 = fast_exp2(m_run[0] - mn0), a1 = fast_exp2(m_run[1] - mn1);
        l_run[0] *= a0;
        l_run[1] *= a1;
        oacc[0] *= a0;
        oacc[1] *= a1;
#pragma unroll
        for (int mt = 0; mt < 8; ++mt) {
          acc[mt][0] *= a0; acc[mt][1] *= a1; acc[mt][2] *= a0; acc[mt][3] *= a1;
        }
        m_run[0] = mn0;
        m_run[1] = mn1;
      }
      const float p0 = fast_exp2(s2[0] - m_run[0]), p1 = fast_exp2(s2[1] - m_run[1]);
      const float p2 = fast_exp2(s2[2] - m_run[0]), p3 = fast_exp2(s2[3] - m_run[1]);
      l_run[0] += p0 + p2;
      l_run[1] += p1 + p3;
      const unsigned b0 = movmatrix_trans(pack_qt2<QT>(p0, p1));
      const unsigned b1 = movmatrix_trans(pack_qt2<QT>(p2, p3));
      if (VK) {
#pragma unroll
        for (int wg = 0; wg < 4; ++wg) {
          const uint2 A = vrow2[wg][0], Bv = vrow2[wg][1], C = vrow2[wg][2], Dv = vrow2[wg][3];
          const unsigned av[2] = {A.x, A.y}, bv[2] = {Bv.x, Bv.y}, cv[2] = {C.x, C.y}, dv[2] = {Dv.x, Dv.y};
#pragma unroll
          for (int pp = 0; pp < 2; ++pp) {
            mma_qt<QT>(acc[wg * 2 + pp], __byte_perm(av[pp], bv[pp], 0x5410u), __byte_perm(av[pp], bv[pp], 0x7632u),
                       __byte_perm(cv[pp], dv[pp], 0x5410u), __byte_perm(cv[pp], dv[pp], 0x7632u), b0, b1);
          }
        }
      } else {
#pragma unroll
      for (int gr = 0; gr < 2; ++gr) {
        const uint4 A = vrow[gr][0], Bv = vrow[gr][1], C = vrow[gr][2], Dv = vrow[gr][3];
        const unsigned av[4] = {A.x, A.y, A.z, A.w}, bv[4] = {Bv.x, Bv.y, Bv.z, Bv.w};
        const unsigned cv[4] = {C.x, C.y, C.z, C.w}, dv[4] = {Dv.x, Dv.y, Dv.z, Dv.w};
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          mma_qt<QT>(acc[gr * 4 + q], __byte_perm(av[q], bv[q], 0x5410u), __byte_perm(av[q], bv[q], 0x7632u),
                     __byte_perm(cv[q], dv[q], 0x5410u), __byte_perm(cv[q], dv[q], 0x7632u), b0, b1);
        }
      }
      }
    }
  }

  };

  // ---------------------------------------------------------------- packed history
  if (pb > pa) {
    const int n_my = (int)(pb - pa);
    int pf_block = (int)(pa / spb), pf_slice = (int)(pa % spb);   // prefetch cursor
    BlockPtrs pf_ptrs = locate_block<MODE, VK, VG>(P, d_table, d_roles, d_pool, d_pages, d_pool_pages, pf_block, h, d_vroles);
    int to_issue = n_my, issue_stage = 0;
    int meta_block = -1;        // block whose metadata is staged (or in flight) in wmeta
    int folded_block = -2;      // last block whose weights were derived from wmeta
    auto stage_meta = [&](const BlockPtrs& bp, unsigned char* dst, int slot = 0) {
      cp_async16(dst + lane * 16, bp.ks + lane * 16);
      if (lane < (MODE == 0 ? 8 : 16)) cp_async16(dst + 512 + lane * 16, bp.kr + lane * 16);
      for (int i = lane; i < n_pad; i += 32) cp_async4(dst + 768 + i * 4, bp.kpad + i * 4);
      if (VK == 1) {
        unsigned char* const vdst = wvmeta + slot * kValueMeta;
        cp_async16(vdst + lane * 16, bp.vs + lane * 16);
        if (lane < 8) cp_async16(vdst + 512 + lane * 16, bp.vr + lane * 16);
        if (lane < 16) cp_async4(vdst + 640 + lane * 4, bp.vo + lane * 4);
      }
    };
    // FAST: this lane's source pointers of the next slice to request (K rows, V rows, V scale and
    // offset pairs), the shared-memory address of the stage it goes to, slices left in its block
    const unsigned char* fk = pf_ptrs.kp + pf_slice * 2048 + lane * 16;
    const unsigned char* fv = pf_ptrs.vp + pf_slice * (VK ? 2048 : 1024) + lane * 16;
    constexpr int kParamLane = VK != 1 && VG == 4 ? 8 : 4;   // bytes of a parameter array one lane copies per slice
    const unsigned char* fs = pf_ptrs.vs + pf_slice * (kStageP / 2) + lane * kParamLane;
    const unsigned char* fo = pf_ptrs.vo + pf_slice * (kStageP / 2) + lane * kParamLane;
    const unsigned ring_lo = smem_addr(ring), ring_hi = ring_lo + kStages * kStageBytes;
    unsigned issue_addr = ring_lo;
    int pf_left = spb - pf_slice;
    // value rows in a stage.  2-bit values: 32 B per token, the halves of tokens 4..7 (mod 8) swapped.
    // Coded values: 64 B per token like the keys, the 16-byte chunks XORed with (token / 2) % 4 so that
    // the later ldmatrix reads of eight tokens' chunks fall into distinct banks.
    const unsigned fast_v_dst = VK ? (unsigned)(kStageK + (lane >> 2) * 64 + (((lane & 3) ^ ((lane >> 3) & 3)) << 4))
                                   : (unsigned)(kStageK + (((lane >> 1) * 2 + ((lane & 1) ^ ((lane >> 3) & 1))) << 4));
    if (FAST) stage_meta(pf_ptrs, wmeta + (pf_block & 1) * 1024, pf_block & 1);   // the first block's metadata rides with its first slice
    auto issue = [&]() {
      if (FAST) {
        if (to_issue > 0) {
          const unsigned dk = issue_addr + lane * 16, dv = issue_addr + fast_v_dst;
          const unsigned dp = issue_addr + kStageK + kStageV + lane * (VK != 1 && VG == 4 ? 8 : 4);
          asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dk), "l"(fk));
          asm volatile("cp.async.cg.shared.global [%0+512], [%1+512], 16;" ::"r"(dk), "l"(fk));
          asm volatile("cp.async.cg.shared.global [%0+1024], [%1+1024], 16;" ::"r"(dk), "l"(fk));
          asm volatile("cp.async.cg.shared.global [%0+1536], [%1+1536], 16;" ::"r"(dk), "l"(fk));
          asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dv), "l"(fv));
          asm volatile("cp.async.cg.shared.global [%0+512], [%1+512], 16;" ::"r"(dv), "l"(fv));
          if (VK) {
            asm volatile("cp.async.cg.shared.global [%0+1024], [%1+1024], 16;" ::"r"(dv), "l"(fv));
            asm volatile("cp.async.cg.shared.global [%0+1536], [%1+1536], 16;" ::"r"(dv), "l"(fv));
          }
          if (VK != 1 && VG == 4) {
            asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(dp), "l"(fs));
            asm volatile("cp.async.ca.shared.global [%0+256], [%1], 8;" ::"r"(dp), "l"(fo));
          } else if (VK != 1 && VG == 1) {
            if (lane < 16) {
              asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dp), "l"(fs));
              asm volatile("cp.async.ca.shared.global [%0+64], [%1], 4;" ::"r"(dp), "l"(fo));
            }
          } else if (VK != 1) {
            asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dp), "l"(fs));
            asm volatile("cp.async.ca.shared.global [%0+128], [%1], 4;" ::"r"(dp), "l"(fo));
          }
          fk += 2048; fv += VK ? 2048 : 1024; fs += kStageP / 2; fo += kStageP / 2;
          --to_issue;
          issue_addr += kStageBytes;
          if (issue_addr == ring_hi) issue_addr = ring_lo;
          if (--pf_left == 0) {
            pf_left = spb;
            ++pf_block;
            if (to_issue > 0) {
              // the cursor enters a new block: its rows, and its metadata at once into slot block % 2.
              // The cursor runs at most three slices ahead of the slice being consumed and a block has
              // at least two, so the slot's previous block lies behind the consumed one or is the
              // consumed one, whose fold precedes this request (the copies are issued after it).
              pf_ptrs = locate_block<MODE, VK, VG>(P, d_table, d_roles, d_pool, d_pages, d_pool_pages, pf_block, h, d_vroles);
              fk = pf_ptrs.kp + lane * 16; fv = pf_ptrs.vp + lane * 16; fs = pf_ptrs.vs + lane * kParamLane; fo = pf_ptrs.vo + lane * kParamLane;
              stage_meta(pf_ptrs, wmeta + (pf_block & 1) * 1024, pf_block & 1);
            }
          }
        }
        cp_async_commit();
        return;
      }
      if (to_issue > 0) {
        unsigned char* const stage_ptr = ring + issue_stage * kStageBytes;
        if (kMetaInStage) {
          // every slice is a whole block: its metadata travels in the slice's own stage
          stage_meta(pf_ptrs, stage_ptr + kMetaOffset);
        } else {
          // a new block's metadata rides in the same group as its first slice, provided the
          // staging area is no longer needed by an earlier block
          const bool first_of_block = to_issue == n_my || pf_slice == 0;
          if (first_of_block && (meta_block < 0 || folded_block == meta_block)) {
            stage_meta(pf_ptrs, wmeta);
            meta_block = pf_block;
          }
        }
        stage_slice<kSub>(stage_ptr, pf_ptrs.kp, pf_ptrs.vp, pf_ptrs.vs, pf_ptrs.vo, pf_slice * kSliceTokens, T, lane);
        --to_issue;
        if (++issue_stage == kStages) issue_stage = 0;
        if (++pf_slice == spb) {
          pf_slice = 0;
          ++pf_block;
          if (to_issue > 0) pf_ptrs = locate_block<MODE, VK, VG>(P, d_table, d_roles, d_pool, d_pages, d_pool_pages, pf_block, h, d_vroles);
        }
      }
      cp_async_commit();
    };
#pragma unroll
    for (int s = 0; s < kStages - 1; ++s) issue();
    // the dense slices of this warp hide behind the DRAM latency of the first packed slices;
    // their contribution is brought into the packed loop's per-row units (powers of two)
    dense_part();
    if (VK == 2) {
      // 4-bit values: rows r carry nibbles at bit 0 (2^-24), rows r + 8 nibbles at bit 4 (2^-20)
#pragma unroll
      for (int mt = 0; mt < 8; ++mt) {
        acc[mt][0] *= 1.f / 16777216.f;
        acc[mt][1] *= 1.f / 16777216.f;
        acc[mt][2] *= 1.f / 1048576.f;
        acc[mt][3] *= 1.f / 1048576.f;
      }
    }
    if (!VK) {
      const float ix[4] = {1.f / 16777216.f, 1.f / 1048576.f, 1.f / 65536.f, 1.f / 4194304.f};
      const float iy[4] = {1.f / 4194304.f, 1.f / 262144.f, 1.f / 16777216.f, 1.f / 1048576.f};
#pragma unroll
      for (int mt = 0; mt < 8; ++mt) {
        acc[mt][0] *= ix[mt & 3];
        acc[mt][1] *= ix[mt & 3];
        acc[mt][2] *= iy[mt & 3];
        acc[mt][3] *= iy[mt & 3];
      }
    }

    int cur_block = (int)(pa / spb), cur_slice = (int)(pa % spb);
    bool need_weights = true;
    float alpha[2] = {0.f, 0.f}, beta[2] = {0.f, 0.f}, bm[2] = {0.f, 0.f};   // bm = beta - m_run
    const unsigned vsel = (r & 1) ? 0x7632u : 0x5410u;
    // ldmatrix row address of this lane inside a stage's V area: lanes 0-7 / 8-15 name tokens 0-7 /
    // 8-15 of value group 0, lanes 16-31 the same tokens of group 1 (halves of tokens 4..7 swapped)
    const int v_tok = (lane & 7) + 8 * ((lane >> 3) & 1);
    const unsigned v_ldsm = (unsigned)((2 * v_tok + ((lane >> 4) ^ ((v_tok >> 2) & 1))) << 4);
    const unsigned ring_addr = smem_addr(ring), lane16 = lane * 16;
    const unsigned ww_addr = smem_addr(wW) + lane * 8, sel_addr = smem_addr(wsel) + lane * 8;
    int stage_index = 0;
    unsigned consume_addr = ring_lo;
    // coded values: sums of the current block alone (in subnormal units) and of its probabilities
    float bacc[8][4], l_blk[2] = {0.f, 0.f};
#pragma unroll
    for (int mt = 0; mt < 8; ++mt)
#pragma unroll
      for (int k = 0; k < 4; ++k) bacc[mt][k] = 0.f;
    // ldmatrix row addresses inside a stage's value area: lanes 0-7 / 8-15 name tokens 0-7 / 8-15 of
    // the first 16-byte chunk (words 0-7: channels 0-31), lanes 16-31 the same tokens of the second;
    // the other address serves chunks 2 and 3.  Chunks are stored XORed with (token / 2) % 4.
    const int vk_tok = (lane & 7) + 8 * ((lane >> 3) & 1), vk_sw = (vk_tok >> 1) & 3;
    const unsigned vk_ldsm_a = (unsigned)(vk_tok * 64 + (((lane >> 4) ^ vk_sw) << 4));
    const unsigned vk_ldsm_b = (unsigned)(vk_tok * 64 + ((((lane >> 4) + 2) ^ vk_sw) << 4));
    // End of a block (or of this warp's range): the block's sums enter the running output with the
    // block's per-channel scales.  Entry i of a lane's tables is channel 32 (i / 4) + 4 r + i % 4.
    auto flush_values = [&]() {
      float lb0 = l_blk[0], lb1 = l_blk[1];
#pragma unroll
      for (int off = 4; off < 32; off <<= 1) {
        lb0 += __shfl_xor_sync(0xffffffffu, lb0, off);
        lb1 += __shfl_xor_sync(0xffffffffu, lb1, off);
      }
      const int4 kinds4 = *(const int4*)(wvkind + r * 16);
      const int kinds[4] = {kinds4.x, kinds4.y, kinds4.z, kinds4.w};
      // donor slots hold the low nibbles of salient codes: their sums go to the lanes of those channels
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const int kind = (int)(signed char)((kinds[i >> 2] >> (8 * (i & 3))) & 0xff);
        const int mt = 2 * (i >> 2) + ((i >> 1) & 1), x = i & 1;
        if (kind >= 16) {
          const float unit = x ? 1048576.f : 16777216.f;
          *(float2*)(wvx + (kind - 16) * 8 + 2 * j) = make_float2(bacc[mt][2 * x] * unit, bacc[mt][2 * x + 1] * unit);
        }
      }
      __syncwarp();
#pragma unroll
      for (int q4 = 0; q4 < 4; ++q4) {
        const float4 w4 = *(const float4*)(wvw + r * 16 + 4 * q4), k4 = *(const float4*)(wvk + r * 16 + 4 * q4);
        const float wv[4] = {w4.x, w4.y, w4.z, w4.w}, kv[4] = {k4.x, k4.y, k4.z, k4.w};
#pragma unroll
        for (int ii = 0; ii < 4; ++ii) {
          const int i = 4 * q4 + ii;
          const int kind = (int)(signed char)((kinds[q4] >> (8 * ii)) & 0xff);
          const int mt = 2 * q4 + (ii >> 1), x = ii & 1;
          float add0 = fmaf(wv[ii], bacc[mt][2 * x], kv[ii] * lb0), add1 = fmaf(wv[ii], bacc[mt][2 * x + 1], kv[ii] * lb1);
          if (kind >= 0 && kind < 16) {
            const float2 low = *(const float2*)(wvx + kind * 8 + 2 * j);
            const float s_src = kv[ii] * (-1.f / 128.f);
            add0 = fmaf(s_src, low.x, add0);
            add1 = fmaf(s_src, low.y, add1);
          }
          acc[mt][2 * x] += add0;
          acc[mt][2 * x + 1] += add1;
          bacc[mt][2 * x] = 0.f;
          bacc[mt][2 * x + 1] = 0.f;
          (void)i;
        }
      }
      l_blk[0] = l_blk[1] = 0.f;
      __syncwarp();
    };

    for (int it = 0; it < n_my; ++it) {
      cp_async_wait<kStages - 2>();
      __syncwarp();
      // With fewer than three slices per block the next block's metadata can only be staged once
      // this block's fold has released the staging area: there the copies are issued after the
      // fold.  Otherwise they go out first.
      // FAST: a request that enters a new block also requests that block's metadata, possibly into
      // the slot of this slice's block, so the fold of this block (it reads that slot) comes first
      const bool issue_late = FAST ? need_weights : (!kMetaInStage && spb < 3 && need_weights);
      if (!issue_late) issue();

      if (need_weights) {
        // ---- fold this block's descriptor, scales and padding into the query
        unsigned char* meta = wmeta;
        if (FAST) {
          meta = wmeta + (cur_block & 1) * 1024;
        } else if (kMetaInStage) {
          meta = ring + stage_index * kStageBytes + kMetaOffset;
        } else if (meta_block != cur_block) {
          // not prefetched (very short blocks): fetch now and wait for it alone
          BlockPtrs cb = locate_block<MODE, VK, VG>(P, d_table, d_roles, d_pool, d_pages, d_pool_pages, cur_block, h, d_vroles);
          __syncwarp();
          stage_meta(cb, wmeta);
          cp_async_commit();
          cp_async_wait<0>();
          meta_block = cur_block;
          __syncwarp();
        }
        folded_block = cur_block;
        // step 1: this lane owns the four channels c0, c0+1, c0+4, c0+5 (c0 = 8 (lane / 2) + 2 (lane % 2)):
        // exactly the channels of one B-fragment entry (K step 2 ((lane / 2) % 4) + lane % 2, chunk lane / 8)
        const unsigned char* meta_roles = meta + 512;
        const int c0 = 8 * (lane >> 1) + 2 * (lane & 1);
        int role[4], sidx[4];
        float scv[4], fv[4];
        {
          const float2 sa = *(const float2*)(meta + c0 * 4), sb = *(const float2*)(meta + c0 * 4 + 16);
          scv[0] = sa.x; scv[1] = sa.y; scv[2] = sb.x; scv[3] = sb.y;
          if (MODE == 0) {
            const unsigned ba = *(const unsigned short*)(meta_roles + c0), bb = *(const unsigned short*)(meta_roles + c0 + 4);
            role[0] = (int)(signed char)(ba & 0xff);
            role[1] = (int)(signed char)(ba >> 8);
            role[2] = (int)(signed char)(bb & 0xff);
            role[3] = (int)(signed char)(bb >> 8);
          } else {
            const unsigned ba = *(const unsigned*)(meta_roles + c0 * 2), bb = *(const unsigned*)(meta_roles + c0 * 2 + 8);
            role[0] = (int)(short)(ba & 0xffff);
            role[1] = (int)(short)(ba >> 16);
            role[2] = (int)(short)(bb & 0xffff);
            role[3] = (int)(short)(bb >> 16);
          }
        }
        // the block's scales are brought into [0, 2) by a power of two
        unsigned top = __float_as_uint(fmaxf(fmaxf(fabsf(scv[0]), fabsf(scv[1])), fmaxf(fabsf(scv[2]), fabsf(scv[3]))));
        top = __reduce_max_sync(0xffffffffu, top);
        const int ex_f = max(-60, min(60, (int)(top >> 23) - 127));
        const float down = __uint_as_float((unsigned)(127 - ex_f) << 23);
        bool bad = false;
        float* const pads = (float*)(meta + 768);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          if (role[i] > 127 || role[i] < -1 - n_pad) {
            bad = true;
            role[i] = -1;
          }
          sidx[i] = -1;
          // the odd channel of a byte is its high nibble: 16 times the code as an fp16 subnormal
          fv[i] = scv[i] * ((i & 1) ? 0.0625f * down : down);
          if (role[i] >= 0) {
            // salient: both of its slots leave the linear fold (its exact, dtype-rounded value is
            // rebuilt per token); its index in the padding list is recorded in its donor's role
            fv[i] = 0.f;
            const int idx = -(MODE == 0 ? (int)((const signed char*)meta_roles)[role[i]] : (int)((const short*)meta_roles)[role[i]]) - 2;
            if (idx >= 0 && idx < n_pad) sidx[i] = idx; else bad = true;
          } else if (role[i] < -1) {
            // donor: its slot holds the low nibble of a salient code; the reference stores the
            // sampled mean as the channel's own value and rounds it to the model dtype (in place:
            // one donor per list entry)
            fv[i] = 0.f;
            pads[-role[i] - 2] = to_float<QT>(from_float<QT>(pads[-role[i] - 2]));
          }
        }
        if (bad) atomicOr(P.status, INQ_STATUS_BAD_INDEX);
        *(uint2*)(wfrag + ((2 * ((lane >> 1) & 3) + (lane & 1)) * 4 + (lane >> 3)) * 8) =
            make_uint2(pack_half2(fv[0], fv[2]), pack_half2(fv[1], fv[3]));
        // the selection cells of the last block are cleared through their recorded offsets
        for (int v = lane; v < 2 * n_pad; v += 32) *(unsigned short*)(wsel + wcell[v]) = 0;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          if (sidx[i] >= 0) {
            const int idx = sidx[i];
            wsrc[idx] = (unsigned char)(c0 + (i & 1) + 4 * (i >> 1));
            wdon[idx] = (unsigned char)role[i];
            // in the units of the score accumulator (see the salient query entries below); the second
            // code of a gather column carries a factor 1/512
            wssc[idx] = scv[i] * (down * ((idx & 8) ? 0.125f : (1.f / 4096.f)));
          }
        }
        __syncwarp();
        // selection matrix: column (idx & 7) gathers the codes of TWO salient channels into one fp32
        // accumulator, code' = 16 * (high nibble of the source) + (low nibble in the donor slot) of
        // salient idx with weight 2^-13 when idx & 8 is clear and with weight 2^-22 when it is set;
        // every entry and every partial sum is exact.  One cell per lane: entry v is the source
        // (even v) or the donor slot (odd v) of salient v / 2.
        for (int v = lane; v < 2 * n_pad; v += 32) {
          const int idx = v >> 1, which = v & 1;
          const int c = (which ? wdon[idx] : wsrc[idx]) & 127;
          const int jj = c >> 5, u = c & 31;
          const int ks = 2 * (u >> 3) + ((u >> 1) & 1), half = u & 1, e = (u >> 2) & 1;
          const int target = ((idx & 7) << 2) | jj;
          const int cell = ((((idx >> 4) * 8 + ks) * 32 + target) * 8) + half * 4 + e * 2;
          // fp16 bits of 32768 (source), 2048 (donor), each divided by 16 for the high nibble of a
          // byte and by 512 for the second salient channel of the column
          *(unsigned short*)(wsel + cell) = (unsigned short)(0x7800 - (which + half) * 0x1000 - ((idx >> 3) & 1) * 0x2400);
          wcell[v] = (unsigned short)cell;
        }
        // query at the salient channels, as B fragments of the salient step.  The step adds straight
        // into the score accumulator, whose unit is alpha = qinv * 2^(24 + ex_f): the staged query
        // times 2^-12 and the salient value times 2^-(12 + ex_f) give exactly that unit, and both
        // factors are powers of two, so the rounding to the model dtype is the reference's
        {
          for (int gsel = 0; gsel < groups; ++gsel) {
            unsigned short qv[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              const int i = gsel * 16 + 2 * j + (k & 1) + (k >> 1) * 8;
              const int c = wsrc[min(i, 63)];
              const QT qt = from_float<QT>(qs[(r * 4 + (c >> 5)) * kQChunk + (c & 31)] * (1.f / 4096.f));
              qv[k] = i < n_pad ? *(const unsigned short*)&qt : (unsigned short)0;
            }
            *(uint2*)(wqsal + (gsel * 32 + lane) * 8) = make_uint2((unsigned)qv[0] | ((unsigned)qv[1] << 16),
                                                                   (unsigned)qv[2] | ((unsigned)qv[3] << 16));
          }
        }
        // the donors' constant values times the query: lane (r, j) sums the list entries r, r + 8, ...
        // for query heads 2j and 2j+1, the eight rows are then added up
        float dterm0 = 0.f, dterm1 = 0.f;
        for (int i = r; i < n_pad; i += 8) {
          const int c = wdon[i] & 127;
          const float pad = pads[i];
          const float* qd = qs + (2 * j * 4 + (c >> 5)) * kQChunk + (c & 31);
          dterm0 = fmaf(qd[0], pad, dterm0);
          dterm1 = fmaf(qd[4 * kQChunk], pad, dterm1);
        }
#pragma unroll
        for (int off = 4; off < 32; off <<= 1) {
          dterm0 += __shfl_xor_sync(0xffffffffu, dterm0, off);
          dterm1 += __shfl_xor_sync(0xffffffffu, dterm1, off);
        }
        // step 2: the B fragments of the eight K steps are the staged query (fp16 pairs in fragment
        // order) times the block's channel weights, one HMUL2 per register; the same fragments
        // against an A operand of ones (1 for a low nibble, 16 for a high one) give the sum of the
        // weights per query head, i.e. the contribution of the codes' zero point 8
        float wsum[4] = {0.f, 0.f, 0.f, 0.f};
        {
          const unsigned qf_addr = launder(smem_addr(qfrag) + lane * 8), ff_addr = launder(smem_addr(wfrag) + j * 8);
#define INQ_FOLD(KS)                                                                                       \
  {                                                                                                        \
    const uint2 qq = lds64<(KS) * 256>(qf_addr), ff2 = lds64<(KS) * 32>(ff_addr);                          \
    const uint2 ww = make_uint2(hmul2_bits(qq.x, ff2.x), hmul2_bits(qq.y, ff2.y));                         \
    *(uint2*)(wW + ((KS) * 32 + lane) * 8) = ww;                                                           \
    mma_f16(wsum, 0x00010001u, 0x00010001u, 0x00100010u, 0x00100010u, ww.x, ww.y);                         \
  }
          INQ_FOLD(0) INQ_FOLD(1) INQ_FOLD(2) INQ_FOLD(3) INQ_FOLD(4) INQ_FOLD(5) INQ_FOLD(6) INQ_FOLD(7)
#undef INQ_FOLD
        }
        // raw score -> base-2 score: undo 2^-24 (subnormal nibbles), the scale exponent and the query
        // factor; score columns of this thread are query heads 2j and 2j+1
        {
          const float2 qf = *(const float2*)(qinv + 2 * j);
          const float up = __uint_as_float((unsigned)(127 + 24 + ex_f) << 23);
          alpha[0] = qf.x * up;
          alpha[1] = qf.y * up;
          beta[0] = fmaf(-8.f * alpha[0], wsum[0], qf.x * dterm0);
          beta[1] = fmaf(-8.f * alpha[1], wsum[1], qf.y * dterm1);
        }
        bm[0] = beta[0] - m_run[0];
        bm[1] = beta[1] - m_run[1];
        if (VK == 1) {
          // flush tables of the value block: lane (r, j) derives entries 4j .. 4j+3 of row r
          const unsigned char* const vmeta = wvmeta + (cur_block & 1) * kValueMeta;
          const float* const vscale = (const float*)vmeta;
          const signed char* const vroles = (const signed char*)(vmeta + 512);
          const float* const vpads = (const float*)(vmeta + 640);
          bool vbad = false;
#pragma unroll
          for (int ii = 0; ii < 4; ++ii) {
            const int c = 32 * j + 4 * r + ii;
            const float sc = vscale[c];
            const float unit = (ii & 1) ? 1048576.f : 16777216.f;
            int role = vroles[c];
            float w = sc * unit, k = -8.f * sc;
            int kind = -1;
            if (role > 127 || role < -17) {
              vbad = true;
              w = 0.f; k = 0.f;
            } else if (role >= 0) {
              const int idx = -(int)vroles[role] - 2;
              if (idx >= 0 && idx < 16) {
                kind = idx;
                w = 16.f * sc * unit;
                k = -128.f * sc;
              } else {
                vbad = true;
                w = 0.f; k = 0.f;
              }
            } else if (role < -1) {
              kind = 16 + (-role - 2);
              w = 0.f;
              k = to_float<QT>(from_float<QT>(vpads[-role - 2]));
            }
            wvw[r * 16 + 4 * j + ii] = w;
            wvk[r * 16 + 4 * j + ii] = k;
            wvkind[r * 16 + 4 * j + ii] = (signed char)kind;
          }
          if (vbad) atomicOr(P.status, INQ_STATUS_BAD_INDEX);
        }
        need_weights = false;
        if (issue_late) {
          __syncwarp();   // every lane has read the per-channel terms: the staging area is free
          issue();
        }
      }

      const unsigned stage = launder(FAST ? consume_addr : ring_addr + stage_index * kStageBytes);
      const unsigned ww_it = launder(ww_addr), sel_it = launder(sel_addr);
      if (FAST) {
        consume_addr += kStageBytes;
        if (consume_addr == ring_hi) consume_addr = ring_lo;
      } else if (++stage_index == kStages) {
        stage_index = 0;
      }
      // ---- scores of two 16-token sub-slices (tokens 0..15 and 16..31 of the stage): K nibbles
      //      times the folded query, plus the exactly rebuilt salient channels
      float S[2][4];
      {
        // C[sub-slice][frag]: column n of the gather holds the codes of salient n and n + 8 of the
        // group as (code'_n - 128) + (code'_{n+8} - 128) / 512, in units of 2^-13
        float C[2][4];
        // One sub-slice at a time keeps the live register set small: this lane's 16 bytes
        // (channels 32j..32j+31) of tokens r and r+8 of the sub-slice.
// One K step: the fragments of the NEXT step are fetched before this step's MMAs are issued,
// so no MMA waits on a shared-memory load that was issued just before it.
#define INQ_KMMA(U, X, Y, FIRST, WQ, F)                                                                   \
  {                                                                                                       \
    const unsigned a0 = (X) & 0x000F000Fu, a1 = (Y) & 0x000F000Fu, a2 = (X) & 0x00F000F0u, a3 = (Y) & 0x00F000F0u; \
    if (FIRST) mma_f16_first(S[U], a0, a1, a2, a3, WQ.x, WQ.y);                                           \
    else mma_f16(S[U], a0, a1, a2, a3, WQ.x, WQ.y);                                                       \
    if (SAL) {                                                                                            \
      if (FIRST) mma_f16_init(C[U], a0, a1, a2, a3, F.x, F.y, kGatherInit);                               \
      else mma_f16(C[U], a0, a1, a2, a3, F.x, F.y);                                                       \
    }                                                                                                     \
  }
#define INQ_KSTEP(KS, M, SH, FIRST, WQ, F, WQN, FN)                                                       \
  {                                                                                                       \
    if ((KS) < 7) {                                                                                       \
      WQN = lds64<(((KS) + 1) & 7) * 256>(ww_it);                                                         \
      if (SAL) FN = lds64<(((KS) + 1) & 7) * 256>(sel_it);                                                \
    }                                                                                                     \
    INQ_KMMA(0, kx0.M >> SH, ky0.M >> SH, FIRST, WQ, F)                                                   \
    if (kSub > 1) INQ_KMMA(kSub - 1, kx1.M >> SH, ky1.M >> SH, FIRST, WQ, F)                              \
  }
        {
          const uint4 kx0 = lds128<0>(stage + lane16), ky0 = lds128<512>(stage + lane16);
          const uint4 kx1 = lds128<(kSub > 1 ? 1024 : 0)>(stage + lane16), ky1 = lds128<(kSub > 1 ? 1536 : 512)>(stage + lane16);
          uint2 wa = lds64<0>(ww_it), wb_;
          uint2 fa = make_uint2(0u, 0u), fb = fa;
          if (SAL) fa = lds64<0>(sel_it);
          INQ_KSTEP(0, x, 0, true, wa, fa, wb_, fb)
          INQ_KSTEP(1, x, 8, false, wb_, fb, wa, fa)
          INQ_KSTEP(2, y, 0, false, wa, fa, wb_, fb)
          INQ_KSTEP(3, y, 8, false, wb_, fb, wa, fa)
          INQ_KSTEP(4, z, 0, false, wa, fa, wb_, fb)
          INQ_KSTEP(5, z, 8, false, wb_, fb, wa, fa)
          INQ_KSTEP(6, w, 0, false, wa, fa, wb_, fb)
          INQ_KSTEP(7, w, 8, false, wb_, fb, wa, fa)
        }
#undef INQ_KMMA
#undef INQ_KSTEP
        if (SAL) {
          for (int gsel = 0; gsel < groups; ++gsel) {
            if (gsel) {
              // further groups of 16 salient channels (salient fractions above 1/8)
              const uint4 k0 = lds128<0>(stage + lane16), k1 = lds128<512>(stage + lane16);
              const uint4 k2 = lds128<(kSub > 1 ? 1024 : 0)>(stage + lane16), k3 = lds128<(kSub > 1 ? 1536 : 512)>(stage + lane16);
              const unsigned kw[4][4] = {{k0.x, k0.y, k0.z, k0.w}, {k1.x, k1.y, k1.z, k1.w},
                                         {k2.x, k2.y, k2.z, k2.w}, {k3.x, k3.y, k3.z, k3.w}};
#pragma unroll
              for (int u = 0; u < kSub; ++u)
#pragma unroll
                for (int k = 0; k < 4; ++k) C[u][k] = kGatherInit;
              const uint2* selg = (const uint2*)wsel + gsel * 256 + lane;
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                unsigned x0 = kw[0][i], y0 = kw[1][i], x1 = kw[2][i], y1 = kw[3][i];
#pragma unroll
                for (int hh = 0; hh < 2; ++hh) {
                  const uint2 f = selg[(2 * i + hh) * 32];
                  mma_f16(C[0], x0 & 0x000F000Fu, y0 & 0x000F000Fu, x0 & 0x00F000F0u, y0 & 0x00F000F0u, f.x, f.y);
                  if (kSub > 1)
                    mma_f16(C[kSub - 1], x1 & 0x000F000Fu, y1 & 0x000F000Fu, x1 & 0x00F000F0u, y1 & 0x00F000F0u, f.x, f.y);
                  x0 >>= 8; y0 >>= 8; x1 >>= 8; y1 >>= 8;
                }
              }
            }
            // value = fl32((code' - 128) * scale) rounded to the model dtype, as the reference's
            // dequantised tensor holds it.  The two codes of an accumulator are separated exactly:
            // adding 1.5 * 2^23 rounds to the integer part (the fraction stays within 1/4), the rest
            // is the second code over 512.
            const float2 sc0 = *(const float2*)(wssc + gsel * 16 + 2 * j);
            const float2 sc1 = *(const float2*)(wssc + gsel * 16 + 8 + 2 * j);
            const uint2 qb = *(const uint2*)(wqsal + (gsel * 32 + lane) * 8);
#pragma unroll
            for (int u = 0; u < kSub; ++u) {
              float hi[4], lo[4];
#pragma unroll
              for (int k = 0; k < 4; ++k) {
                hi[k] = fmaf(C[u][k], 8192.f, 12582912.f) - 12582912.f;
                lo[k] = fmaf(C[u][k], 8192.f, -hi[k]);
              }
              const unsigned a0 = pack_qt2<QT>(hi[0] * sc0.x, hi[1] * sc0.y);
              const unsigned a1 = pack_qt2<QT>(hi[2] * sc0.x, hi[3] * sc0.y);
              const unsigned a2 = pack_qt2<QT>(lo[0] * sc1.x, lo[1] * sc1.y);
              const unsigned a3 = pack_qt2<QT>(lo[2] * sc1.x, lo[3] * sc1.y);
              mma_qt<QT>(S[u], a0, a1, a2, a3, qb.x, qb.y);
            }
          }
        }
      }
      // s2[u][k]: sub-slice u; k = 0,1 -> token r (+16u), heads 2j, 2j+1; k = 2,3 -> token r+8 (+16u)
      float s2[2][4];
#pragma unroll
      for (int u = 0; u < kSub; ++u) {
        // relative to the running reference maximum: bm = beta - m_run
        s2[u][0] = fmaf(S[u][0], alpha[0], bm[0]);
        s2[u][1] = fmaf(S[u][1], alpha[1], bm[1]);
        s2[u][2] = fmaf(S[u][2], alpha[0], bm[0]);
        s2[u][3] = fmaf(S[u][3], alpha[1], bm[1]);
      }
      if (FAST) {
        // whole slices only: the one mask left is the packed copy of the tokens the exact sink holds
        const int g0 = cur_block * T + cur_slice * kSliceTokens;
        if (g0 < first_visible) {
#pragma unroll
          for (int u = 0; u < kSub; ++u) {
            if (g0 + 16 * u + r < first_visible) s2[u][0] = s2[u][1] = -INFINITY;
            if (g0 + 16 * u + r + 8 < first_visible) s2[u][2] = s2[u][3] = -INFINITY;
          }
        }
      } else {
        const int tok0 = cur_slice * kSliceTokens;
        const long long g0 = (long long)cur_block * T + tok0;
        if (tok0 + kSliceTokens > T || g0 < first_visible) {
#pragma unroll
          for (int u = 0; u < kSub; ++u) {
            const int t_lo = tok0 + 16 * u + r, t_hi = t_lo + 8;
            if (!(t_lo < T && g0 + 16 * u + r >= first_visible)) s2[u][0] = s2[u][1] = -INFINITY;
            if (!(t_hi < T && g0 + 16 * u + r + 8 >= first_visible)) s2[u][2] = s2[u][3] = -INFINITY;
          }
        }
      }
      // ---- online softmax (base 2) over the 32 tokens.  The reference maximum is raised only when
      //      a score exceeds it by more than the slack, so the accumulators are rescaled rarely and
      //      probabilities stay below 2^slack; the common case costs one vote and the scores arrive
      //      already relative to the reference
      {
        float mx0 = fmaxf(s2[0][0], s2[0][2]), mx1 = fmaxf(s2[0][1], s2[0][3]);
        if (kSub > 1) {
          mx0 = fmaxf(mx0, fmaxf(s2[kSub - 1][0], s2[kSub - 1][2]));
          mx1 = fmaxf(mx1, fmaxf(s2[kSub - 1][1], s2[kSub - 1][3]));
        }
        if (__any_sync(0xffffffffu, mx0 > kRescaleSlack || mx1 > kRescaleSlack)) {
          // rare: recompute the absolute scores (the first slice of a warp meets a reference of
          // -1e30, against which the relative form has no precision left), raise the reference
          float ab[2][4];
#pragma unroll
          for (int u = 0; u < kSub; ++u) {
            ab[u][0] = s2[u][0] == -INFINITY ? -INFINITY : fmaf(S[u][0], alpha[0], beta[0]);
            ab[u][1] = s2[u][1] == -INFINITY ? -INFINITY : fmaf(S[u][1], alpha[1], beta[1]);
            ab[u][2] = s2[u][2] == -INFINITY ? -INFINITY : fmaf(S[u][2], alpha[0], beta[0]);
            ab[u][3] = s2[u][3] == -INFINITY ? -INFINITY : fmaf(S[u][3], alpha[1], beta[1]);
          }
          mx0 = fmaxf(ab[0][0], ab[0][2]);
          mx1 = fmaxf(ab[0][1], ab[0][3]);
          if (kSub > 1) {
            mx0 = fmaxf(mx0, fmaxf(ab[kSub - 1][0], ab[kSub - 1][2]));
            mx1 = fmaxf(mx1, fmaxf(ab[kSub - 1][1], ab[kSub - 1][3]));
          }
#pragma unroll
          for (int off = 4; off < 32; off <<= 1) {
            mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, off));
            mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, off));
          }
          const float mn0 = fmaxf(m_run[0], mx0), mn1 = fmaxf(m_run[1], mx1);
          const float a0 = fast_exp2(m_run[0] - mn0), a1 = fast_exp2(m_run[1] - mn1);
          l_run[0] *= a0;
          l_run[1] *= a1;
          oacc[0] *= a0;
          oacc[1] *= a1;
#pragma unroll
          for (int mt = 0; mt < 8; ++mt) {
            acc[mt][0] *= a0; acc[mt][1] *= a1; acc[mt][2] *= a0; acc[mt][3] *= a1;
          }
          if (VK == 1) {
            l_blk[0] *= a0;
            l_blk[1] *= a1;
#pragma unroll
            for (int mt = 0; mt < 8; ++mt) {
              bacc[mt][0] *= a0; bacc[mt][1] *= a1; bacc[mt][2] *= a0; bacc[mt][3] *= a1;
            }
          }
          m_run[0] = mn0;
          m_run[1] = mn1;
          bm[0] = beta[0] - mn0;
          bm[1] = beta[1] - mn1;
#pragma unroll
          for (int u = 0; u < kSub; ++u) {
            s2[u][0] = ab[u][0] - mn0; s2[u][1] = ab[u][1] - mn1;
            s2[u][2] = ab[u][2] - mn0; s2[u][3] = ab[u][3] - mn1;
          }
        }
      }
      float pr[2][4];
#pragma unroll
      for (int u = 0; u < kSub; ++u) {
        pr[u][0] = fast_exp2(s2[u][0]);
        pr[u][1] = fast_exp2(s2[u][1]);
        pr[u][2] = fast_exp2(s2[u][2]);
        pr[u][3] = fast_exp2(s2[u][3]);
        l_run[0] += pr[u][0] + pr[u][2];
        l_run[1] += pr[u][1] + pr[u][3];
      }
      // ---- values: probabilities times the per-token group scale, codes as fp16 subnormals
#define INQ_PV(U)                                                                                          \
  {                                                                                                        \
    /* probabilities as fp16, transposed into B fragments: tokens (2j, 2j+1) and (2j+8, 2j+9) of head r */ \
    const unsigned t0 = movmatrix_trans(pack_half2(pr[U][0], pr[U][1]));                                   \
    const unsigned t1 = movmatrix_trans(pack_half2(pr[U][2], pr[U][3]));                                   \
    const unsigned sp = stage + kStageK + kStageV + 8 * j;                                                 \
    const uint2 s_lo = lds64<64 * (U)>(sp), s_hi = lds64<64 * (U) + 32>(sp);                               \
    const uint2 o_lo = lds64<kStageP / 2 + 64 * (U)>(sp), o_hi = lds64<kStageP / 2 + 64 * (U) + 32>(sp);   \
    /* offsets: rows 0 and 1 of a 16-row MMA are the two value groups */                                   \
    mma_f16(oacc, __byte_perm(o_lo.x, o_lo.y, vsel), 0u, __byte_perm(o_hi.x, o_hi.y, vsel), 0u, t0, t1);   \
    const uint4 M = ldsm4_trans<kStageK + 512 * (U)>(stage + v_ldsm);                                      \
    _Pragma("unroll") for (int gr = 0; gr < 2; ++gr) {                                                     \
      const unsigned gsel2 = gr ? 0x7632u : 0x5410u;                                                       \
      const unsigned b0 = hmul2_bits(t0, __byte_perm(s_lo.x, s_lo.y, gsel2));                              \
      const unsigned b1 = hmul2_bits(t1, __byte_perm(s_hi.x, s_hi.y, gsel2));                              \
      const unsigned M0 = gr ? M.z : M.x, M1 = gr ? M.w : M.y;                                             \
      const unsigned N0 = M0 >> 10, N1 = M1 >> 10;                                                         \
      mma_f16(acc[gr * 4 + 0], M0 & 0x00030003u, M0 & 0x000C000Cu, M1 & 0x00030003u, M1 & 0x000C000Cu, b0, b1); \
      mma_f16(acc[gr * 4 + 1], M0 & 0x00300030u, M0 & 0x00C000C0u, M1 & 0x00300030u, M1 & 0x00C000C0u, b0, b1); \
      mma_f16(acc[gr * 4 + 2], M0 & 0x03000300u, N0 & 0x00030003u, M1 & 0x03000300u, N1 & 0x00030003u, b0, b1); \
      mma_f16(acc[gr * 4 + 3], N0 & 0x000C000Cu, N0 & 0x00300030u, N1 & 0x000C000Cu, N1 & 0x00300030u, b0, b1); \
    }                                                                                                      \
  }
/* 2-bit values with ONE group of 128 channels: a token pair's scales (offsets) are one 32-bit word */     \
#define INQ_PV1(U)                                                                                         \
  {                                                                                                        \
    const unsigned t0 = movmatrix_trans(pack_half2(pr[U][0], pr[U][1]));                                   \
    const unsigned t1 = movmatrix_trans(pack_half2(pr[U][2], pr[U][3]));                                   \
    const unsigned sp = stage + kStageK + kStageV + 4 * j;                                                 \
    const unsigned b0 = hmul2_bits(t0, lds32<32 * (U)>(sp)), b1 = hmul2_bits(t1, lds32<32 * (U) + 16>(sp)); \
    mma_f16(oacc, lds32<kStageP / 2 + 32 * (U)>(sp), 0u, lds32<kStageP / 2 + 32 * (U) + 16>(sp), 0u, t0, t1); \
    const uint4 M = ldsm4_trans<kStageK + 512 * (U)>(stage + v_ldsm);                                      \
    _Pragma("unroll") for (int gr = 0; gr < 2; ++gr) {                                                     \
      const unsigned M0 = gr ? M.z : M.x, M1 = gr ? M.w : M.y;                                             \
      const unsigned N0 = M0 >> 10, N1 = M1 >> 10;                                                         \
      mma_f16(acc[gr * 4 + 0], M0 & 0x00030003u, M0 & 0x000C000Cu, M1 & 0x00030003u, M1 & 0x000C000Cu, b0, b1); \
      mma_f16(acc[gr * 4 + 1], M0 & 0x00300030u, M0 & 0x00C000C0u, M1 & 0x00300030u, M1 & 0x00C000C0u, b0, b1); \
      mma_f16(acc[gr * 4 + 2], M0 & 0x03000300u, N0 & 0x00030003u, M1 & 0x03000300u, N1 & 0x00030003u, b0, b1); \
      mma_f16(acc[gr * 4 + 3], N0 & 0x000C000Cu, N0 & 0x00300030u, N1 & 0x000C000Cu, N1 & 0x00300030u, b0, b1); \
    }                                                                                                      \
  }
/* 2-bit values in FOUR groups of 32 channels: a group is four of the eight 16-bit words of a value MMA's     \
   rows, so every MMA is issued twice, once with rows r < 4 (the others zeroed) against the probabilities     \
   scaled for the lower group and once with rows r >= 4 against those of the upper group */                  \
#define INQ_PV4(U)                                                                                         \
  {                                                                                                        \
    const unsigned t0 = movmatrix_trans(pack_half2(pr[U][0], pr[U][1]));                                   \
    const unsigned t1 = movmatrix_trans(pack_half2(pr[U][2], pr[U][3]));                                   \
    const unsigned sp = stage + kStageK + kStageV + 16 * j;                                                \
    const uint4 sa = lds128<128 * (U)>(sp), sb = lds128<128 * (U) + 64>(sp);                               \
    const uint4 oa = lds128<kStageP / 2 + 128 * (U)>(sp), ob = lds128<kStageP / 2 + 128 * (U) + 64>(sp);   \
    const bool upper = (r & 2) != 0, low_rows = r < 4;                                                     \
    mma_f16(oacc, __byte_perm(upper ? oa.y : oa.x, upper ? oa.w : oa.z, vsel), 0u,                          \
            __byte_perm(upper ? ob.y : ob.x, upper ? ob.w : ob.z, vsel), 0u, t0, t1);                      \
    const uint4 M = ldsm4_trans<kStageK + 512 * (U)>(stage + v_ldsm);                                      \
    _Pragma("unroll") for (int gr = 0; gr < 2; ++gr) {                                                     \
      const unsigned w0 = gr ? sa.y : sa.x, w1 = gr ? sa.w : sa.z, w2 = gr ? sb.y : sb.x, w3 = gr ? sb.w : sb.z; \
      _Pragma("unroll") for (int half = 0; half < 2; ++half) {                                             \
        const unsigned gsel2 = half ? 0x7632u : 0x5410u;                                                   \
        const unsigned b0 = hmul2_bits(t0, __byte_perm(w0, w1, gsel2));                                    \
        const unsigned b1 = hmul2_bits(t1, __byte_perm(w2, w3, gsel2));                                    \
        const bool mine = half ? !low_rows : low_rows;                                                     \
        const unsigned M0 = mine ? (gr ? M.z : M.x) : 0u, M1 = mine ? (gr ? M.w : M.y) : 0u;               \
        const unsigned N0 = M0 >> 10, N1 = M1 >> 10;                                                       \
        mma_f16(acc[gr * 4 + 0], M0 & 0x00030003u, M0 & 0x000C000Cu, M1 & 0x00030003u, M1 & 0x000C000Cu, b0, b1); \
        mma_f16(acc[gr * 4 + 1], M0 & 0x00300030u, M0 & 0x00C000C0u, M1 & 0x00300030u, M1 & 0x00C000C0u, b0, b1); \
        mma_f16(acc[gr * 4 + 2], M0 & 0x03000300u, N0 & 0x00030003u, M1 & 0x03000300u, N1 & 0x00030003u, b0, b1); \
        mma_f16(acc[gr * 4 + 3], N0 & 0x000C000Cu, N0 & 0x00300030u, N1 & 0x000C000Cu, N1 & 0x00300030u, b0, b1); \
      }                                                                                                    \
    }                                                                                                      \
  }
#define INQ_PVK(BASE, LO, HI)                                                                              \
  {                                                                                                        \
    mma_f16(bacc[BASE], (LO) & 0x000F000Fu, (LO) & 0x00F000F0u, (HI) & 0x000F000Fu, (HI) & 0x00F000F0u, t0, t1); \
    const unsigned lo8 = (LO) >> 8, hi8 = (HI) >> 8;                                                       \
    mma_f16(bacc[BASE + 1], lo8 & 0x000F000Fu, lo8 & 0x00F000F0u, hi8 & 0x000F000Fu, hi8 & 0x00F000F0u, t0, t1); \
  }
      if (VK == 2) {
        // 4-bit values in VG groups: the value MMAs of the coded values with the group's per-token
        // scale multiplied into the probabilities; offsets of group r in row r of one more MMA
        constexpr int kPairBytes = 4 * VG;          // parameters of a token pair: 2 tokens x VG groups x fp16
#pragma unroll
        for (int u = 0; u < kSub; ++u) {
          const unsigned t0 = movmatrix_trans(pack_half2(pr[u][0], pr[u][1]));
          const unsigned t1 = movmatrix_trans(pack_half2(pr[u][2], pr[u][3]));
          const unsigned sp = stage + kStageK + kStageV + kPairBytes * j + (u ? 8 * kPairBytes : 0);
          unsigned sc_lo[VG], sc_hi[VG], of_lo, of_hi;   // half2 (token 2j, token 2j+1) and (2j+8, 2j+9) per group
          if (VG == 1) {
            sc_lo[0] = lds32<0>(sp); sc_hi[0] = lds32<4 * kPairBytes>(sp);
            of_lo = lds32<kStageP / 2>(sp); of_hi = lds32<kStageP / 2 + 4 * kPairBytes>(sp);
          } else if (VG == 2) {
            const uint2 a = lds64<0>(sp), b = lds64<4 * kPairBytes>(sp);
            const uint2 c = lds64<kStageP / 2>(sp), d = lds64<kStageP / 2 + 4 * kPairBytes>(sp);
#pragma unroll
            for (int g = 0; g < VG; ++g) {
              sc_lo[g] = __byte_perm(a.x, a.y, g ? 0x7632u : 0x5410u);
              sc_hi[g] = __byte_perm(b.x, b.y, g ? 0x7632u : 0x5410u);
            }
            of_lo = __byte_perm(c.x, c.y, vsel);
            of_hi = __byte_perm(d.x, d.y, vsel);
          } else {
            const uint4 a = lds128<0>(sp), b = lds128<4 * kPairBytes>(sp);
            const uint4 c = lds128<kStageP / 2>(sp), d = lds128<kStageP / 2 + 4 * kPairBytes>(sp);
            const unsigned aw[4] = {a.x, a.y, a.z, a.w}, bw[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
            for (int g = 0; g < VG; ++g) {
              sc_lo[g] = __byte_perm(aw[g >> 1], aw[2 + (g >> 1)], (g & 1) ? 0x7632u : 0x5410u);
              sc_hi[g] = __byte_perm(bw[g >> 1], bw[2 + (g >> 1)], (g & 1) ? 0x7632u : 0x5410u);
            }
            const bool upper = (r & 2) != 0;
            of_lo = __byte_perm(upper ? c.y : c.x, upper ? c.w : c.z, vsel);
            of_hi = __byte_perm(upper ? d.y : d.x, upper ? d.w : d.z, vsel);
          }
          mma_f16(oacc, of_lo, 0u, of_hi, 0u, t0, t1);
          const uint4 Ma = u ? ldsm4_trans<kStageK + 1024>(stage + vk_ldsm_a) : ldsm4_trans<kStageK>(stage + vk_ldsm_a);
          const uint4 Mb = u ? ldsm4_trans<kStageK + 1024>(stage + vk_ldsm_b) : ldsm4_trans<kStageK>(stage + vk_ldsm_b);
          const unsigned lo[4] = {Ma.x, Ma.z, Mb.x, Mb.z}, hi[4] = {Ma.y, Ma.w, Mb.y, Mb.w};
#pragma unroll
          for (int wg = 0; wg < 4; ++wg) {
            const int g = wg * VG / 4;
            const unsigned b0 = hmul2_bits(t0, sc_lo[g]), b1 = hmul2_bits(t1, sc_hi[g]);
            mma_f16(acc[2 * wg], lo[wg] & 0x000F000Fu, lo[wg] & 0x00F000F0u, hi[wg] & 0x000F000Fu, hi[wg] & 0x00F000F0u, b0, b1);
            const unsigned lo8 = lo[wg] >> 8, hi8 = hi[wg] >> 8;
            mma_f16(acc[2 * wg + 1], lo8 & 0x000F000Fu, lo8 & 0x00F000F0u, hi8 & 0x000F000Fu, hi8 & 0x00F000F0u, b0, b1);
          }
        }
      } else if (VK) {
        // coded values: 16 tokens x 32 words of four nibbles each; word w of a token holds channels
        // 4w .. 4w+3, so row r of the MMAs of chunk wg is word 8 wg + r: channels 32 wg + 4 r + (0 | 1)
        // for the nibbles at bit 0 | 4 and, after a shift by 8, + (2 | 3)
#pragma unroll
        for (int u = 0; u < kSub; ++u) {
          const unsigned t0 = movmatrix_trans(pack_half2(pr[u][0], pr[u][1]));
          const unsigned t1 = movmatrix_trans(pack_half2(pr[u][2], pr[u][3]));
          const uint4 Ma = u ? ldsm4_trans<kStageK + 1024>(stage + vk_ldsm_a) : ldsm4_trans<kStageK>(stage + vk_ldsm_a);
          const uint4 Mb = u ? ldsm4_trans<kStageK + 1024>(stage + vk_ldsm_b) : ldsm4_trans<kStageK>(stage + vk_ldsm_b);
          INQ_PVK(0, Ma.x, Ma.y)
          INQ_PVK(2, Ma.z, Ma.w)
          INQ_PVK(4, Mb.x, Mb.y)
          INQ_PVK(6, Mb.z, Mb.w)
          l_blk[0] += pr[u][0] + pr[u][2];
          l_blk[1] += pr[u][1] + pr[u][3];
        }
      } else if (VG == 1) {
        INQ_PV1(0)
        INQ_PV1(1)
      } else if (VG == 4) {
        INQ_PV4(0)
        INQ_PV4(1)
      } else {
      INQ_PV(0)
      if (kSub > 1) INQ_PV(1)
      }
#undef INQ_PV
#undef INQ_PV1
#undef INQ_PV4
#undef INQ_PVK
      if (++cur_slice == spb) {
        cur_slice = 0;
        ++cur_block;
        need_weights = true;
        if (VK == 1) flush_values();
      }
    }
    if (VK == 1 && cur_slice != 0) flush_values();   // this warp's range ended inside a block
    cp_async_wait<0>();
    // a code at bit offset o of its 16-bit lane was multiplied as code * 2^(o-24)
    const float fx[4] = {16777216.f, 1048576.f, 65536.f, 4194304.f};   // offsets 0, 4, 8, 2
    const float fy[4] = {4194304.f, 262144.f, 16777216.f, 1048576.f};  // offsets 2, 6, 0, 4
    if (VK == 2) {
#pragma unroll
      for (int mt = 0; mt < 8; ++mt) {
        acc[mt][0] *= 16777216.f;
        acc[mt][1] *= 16777216.f;
        acc[mt][2] *= 1048576.f;
        acc[mt][3] *= 1048576.f;
      }
    }
#pragma unroll
    for (int mt = 0; mt < (VK ? 0 : 8); ++mt) {
      acc[mt][0] *= fx[mt & 3];
      acc[mt][1] *= fx[mt & 3];
      acc[mt][2] *= fy[mt & 3];
      acc[mt][3] *= fy[mt & 3];
    }
  } else {
    dense_part();
  }

  // ---------------------------------------------------------------- warp -> CTA -> global partial
#pragma unroll
  for (int off = 4; off < 32; off <<= 1) {
    l_run[0] += __shfl_xor_sync(0xffffffffu, l_run[0], off);
    l_run[1] += __shfl_xor_sync(0xffffffffu, l_run[1], off);
  }
  // the offset sums of value group gr, heads 2j and 2j+1, sit in lane (r = gr, j)
  constexpr int kOffsetGroups = VK == 2 || VG == 4 ? VG : 2;
  float osum[kOffsetGroups][2];
#pragma unroll
  for (int gr = 0; gr < kOffsetGroups; ++gr) {
    osum[gr][0] = __shfl_sync(0xffffffffu, oacc[0], gr * 4 + j);
    osum[gr][1] = __shfl_sync(0xffffffffu, oacc[1], gr * 4 + j);
  }
  __syncthreads();   // every warp is done with its ring and weight scratch
  float* wout = (float*)ring;   // [8][132]
#pragma unroll
  for (int mt = 0; mt < 8; ++mt) {
    const int q = mt & 3;
    const int gr = VK == 2 ? (mt >> 1) * VG / 4 : VG == 1 ? 0 : VG == 4 ? 2 * (mt >> 2) + (r >> 2) : mt >> 2;   // value group of the accumulator
    const int ch = VK ? 32 * (mt >> 1) + 4 * r + 2 * (mt & 1) : 64 * (mt >> 2) + 8 * r + 2 * q;
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      const int g = 2 * j + e;
      *(float2*)(wout + g * kRecordStride + ch) = make_float2(acc[mt][e] + osum[gr][e], acc[mt][2 + e] + osum[gr][e]);
    }
  }
  if (r == 0) {
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      wout[(2 * j + e) * kRecordStride + 128] = m_run[e];
      wout[(2 * j + e) * kRecordStride + 129] = l_run[e];
    }
  }
  __syncthreads();
  float* record = P.partials + ((long long)blockIdx.x + pair) * kRecordFloats;
  {
    const int c = threadIdx.x;   // one channel per thread
    const float* w0 = (const float*)(warp_base + (ring - wb));
    const int wstride = warp_bytes / 4;
    for (int g = 0; g < g_valid; ++g) {
      float mw[kWarps], top = kNegBig;
#pragma unroll
      for (int w = 0; w < kWarps; ++w) {
        mw[w] = w0[w * wstride + g * kRecordStride + 128];
        top = fmaxf(top, mw[w]);
      }
      float o = 0.f, l = 0.f;
#pragma unroll
      for (int w = 0; w < kWarps; ++w) {
        const float wt = fast_exp2(mw[w] - top);
        o = fmaf(w0[w * wstride + g * kRecordStride + c], wt, o);
        l = fmaf(w0[w * wstride + g * kRecordStride + 129], wt, l);
      }
      record[g * kRecordStride + c] = o;
      if (c == 0) {
        record[g * kRecordStride + 128] = top;
        record[g * kRecordStride + 129] = l;
      }
    }
  }
  // ---------------------------------------------------------------- last CTA merges
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    const int old = atomicAdd(P.counters + pair, 1);
    s_is_last = (old == n_cta_pair - 1);
    if (s_is_last) P.counters[pair] = 0;   // scratch is left zeroed for the next launch
  }
  __syncthreads();
  if (s_is_last) {
  __threadfence();
    // A sequence decoded alone is cut into a hundred parts per pair, so this merge is written for
    // many loads in flight: (m, l) of every (query head, part) are staged first, the weights
    // come from shared memory, and each thread then sums 8 channels of one head over the parts
    // with 16 vector loads outstanding.
    float* mw = (float*)warp_base;                 // [8][np] running maxima, then weights
    const int np = n_cta_pair;
    float* lw = mw + 8 * np;                       // [8][np] partial normalisers
    float* norm = lw + 8 * np;
    float* mtop = norm + 8;
    const float* base = P.partials + ((long long)first_cta + pair) * kRecordFloats;
    float* const partial = SEQ(partial_out);
#pragma unroll 4
    for (int i = threadIdx.x; i < 8 * np; i += kThreads) {
      const int g = i & 7, p = i >> 3;
      if (g < g_valid) {
        const float2 ml = __ldcg((const float2*)(base + (long long)p * kRecordFloats + g * kRecordStride + 128));
        mw[g * np + p] = ml.x;
        lw[g * np + p] = ml.y;
      }
    }
    __syncthreads();
    for (int g = warp; g < g_valid; g += kWarps) {
      float top = kNegBig;
      for (int p = lane; p < np; p += 32) top = fmaxf(top, mw[g * np + p]);
#pragma unroll
      for (int off = 16; off; off >>= 1) top = fmaxf(top, __shfl_xor_sync(0xffffffffu, top, off));
      float l = 0.f;
      for (int p = lane; p < np; p += 32) {
        const float wt = fast_exp2(mw[g * np + p] - top);
        mw[g * np + p] = wt;
        l = fmaf(lw[g * np + p], wt, l);
      }
#pragma unroll
      for (int off = 16; off; off >>= 1) l += __shfl_xor_sync(0xffffffffu, l, off);
      if (lane == 0) {
        norm[g] = l;
        mtop[g] = top;
      }
    }
    __syncthreads();
    const int g = threadIdx.x >> 4, c8 = (threadIdx.x & 15) * 8;   // kThreads = 128: 8 heads x 16 threads
    float4 ex_a = make_float4(0.f, 0.f, 0.f, 0.f), ex_b = ex_a;
    if (g < g_valid) {
      float o[8];
#pragma unroll
      for (int k = 0; k < 8; ++k) o[k] = 0.f;
      const float* rec = base + g * kRecordStride + c8;
      const float* wg = mw + g * np;
      int p = 0;
      for (; p + 8 <= np; p += 8) {
        float4 va[8], vb[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          va[u] = __ldcg((const float4*)(rec + (long long)(p + u) * kRecordFloats));
          vb[u] = __ldcg((const float4*)(rec + (long long)(p + u) * kRecordFloats) + 1);
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          const float wt = wg[p + u];
          o[0] = fmaf(va[u].x, wt, o[0]); o[1] = fmaf(va[u].y, wt, o[1]); o[2] = fmaf(va[u].z, wt, o[2]); o[3] = fmaf(va[u].w, wt, o[3]);
          o[4] = fmaf(vb[u].x, wt, o[4]); o[5] = fmaf(vb[u].y, wt, o[5]); o[6] = fmaf(vb[u].z, wt, o[6]); o[7] = fmaf(vb[u].w, wt, o[7]);
        }
      }
      for (; p < np; ++p) {
        const float4 va = __ldcg((const float4*)(rec + (long long)p * kRecordFloats));
        const float4 vb = __ldcg((const float4*)(rec + (long long)p * kRecordFloats) + 1);
        const float wt = wg[p];
        o[0] = fmaf(va.x, wt, o[0]); o[1] = fmaf(va.y, wt, o[1]); o[2] = fmaf(va.z, wt, o[2]); o[3] = fmaf(va.w, wt, o[3]);
        o[4] = fmaf(vb.x, wt, o[4]); o[5] = fmaf(vb.y, wt, o[5]); o[6] = fmaf(vb.z, wt, o[6]); o[7] = fmaf(vb.w, wt, o[7]);
      }
      if (P.exchange) {
        // handed to the exchange below (every thread of the CTA takes part in it)
        ex_a = make_float4(o[0], o[1], o[2], o[3]);
        ex_b = make_float4(o[4], o[5], o[6], o[7]);
      } else if (partial) {
        // this rank's share of a sequence split across GPUs: keep the record un-normalised
        float* rec_out = partial + (q_head0 + g) * 130;
#pragma unroll
        for (int k = 0; k < 8; k += 2) *(float2*)(rec_out + c8 + k) = make_float2(o[k], o[k + 1]);
        if (c8 == 0) {
          rec_out[128] = mtop[g];
          rec_out[129] = norm[g];
        }
      } else {
        QT* out = (QT*)SEQ(out) + (q_head0 + g) * 128 + c8;
        const float inv = norm[g];
#pragma unroll
        for (int k = 0; k < 8; ++k) out[k] = from_float<QT>(o[k] / inv);
      }
    }
    if (P.exchange) {
      const bool active = g < g_valid;
      const float top = active ? mtop[g] : 0.f, l = active ? norm[g] : 1.f;
      __syncthreads();   // the merge is done with its shared scratch: it now stages the pair's record
      exchange_pair<QT>(P.exchange, pair, (long long)seq * P.H * P.G + q_head0, g, g_valid, c8, ex_a, ex_b, top, l,
                        (QT*)SEQ(out) + (q_head0 + g) * 128 + c8, P.status, (float*)warp_base);
    }
  }
  __syncthreads();   // shared scratch is reused by the next pair of this CTA
  }  // pairs of this CTA
  if (P.fused_append || P.exchange) {
    // Every CTA has read the tail lengths of the pairs it visited (and the step number of the
    // exchange) by the time it arrives here; the last one to arrive advances them for the next step.
    __shared__ int s_grid_last;
    __syncthreads();
    if (threadIdx.x == 0) {
      __threadfence();
      const int old = atomicAdd(P.counters + P.n_pairs, 1);
      s_grid_last = old == (int)gridDim.x - 1;
      if (s_grid_last) P.counters[P.n_pairs] = 0;
    }
    __syncthreads();
    if (s_grid_last) {
      if (P.fused_append) {
        for (int s = threadIdx.x; s < P.n_seq; s += kThreads) {
          const SeqDesc* d = P.seqs ? P.seqs + s : &P.one;
          if (d->new_k && d->tail_tokens_dev) atomicAdd((int*)d->tail_tokens_dev, 1);
        }
      }
      if (P.exchange && threadIdx.x == 0) P.exchange->epoch[0] += 1;
    }
  }
}

#undef SEQ
static int smem_bytes(int groups, int sub, int vk = 0, int vg = 2) {
  const int stage = vk == 0 && vg == 1 ? SliceCfg<2, 0, 1>::kStageBytes
                  : vk == 0 && vg == 4 ? SliceCfg<2, 0, 4>::kStageBytes
                  : vk == 2 ? (vg == 1 ? SliceCfg<2, 2, 1>::kStageBytes : vg == 2 ? SliceCfg<2, 2, 2>::kStageBytes : SliceCfg<2, 2, 4>::kStageBytes)
                  : vk ? SliceCfg<2, 1>::kStageBytes : (sub == 1 ? SliceCfg<1>::kStageBytes : SliceCfg<2>::kStageBytes);
  return kQBytes + kWarps * warp_smem_bytes(groups, stage, vk == 1);
}

}  // namespace inq

using namespace inq;

// Per-device launch state.  Function attributes, occupancy answers and the SM count belong to a
// device, not to the process: a process that drives several GPUs (or several host threads) gets
// one record per device ordinal, filled under a mutex on first use.
constexpr int kMaxDevices = 64;
constexpr int kKernelVariants = 32;   // 16 general, 4 whole-slice, 2 coded values, 6 4-bit values, 4 2-bit values in one or four groups
struct DeviceState {
  int sm_count = 0;
  bool raised[kKernelVariants] = {};
  int per_sm[kKernelVariants][5] = {};
  void* static_scratch = nullptr;   // resolved address of the allocation-free entry point's array
  bool static_counters_stale = false;
};
static DeviceState g_devices[kMaxDevices];
static std::mutex g_devices_mutex;

static int current_device() {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return -1;
  return dev;
}

static int sm_count() {
  const int dev = current_device();
  if (dev < 0) return 148;
  std::lock_guard<std::mutex> guard(g_devices_mutex);
  DeviceState& d = g_devices[dev];
  if (!d.sm_count) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && n > 0)
      d.sm_count = n;
    else
      return 148;
  }
  return d.sm_count;
}

// Flat decomposition shared by the planner and the launcher.
struct Plan {
  int n_ctas;
  long long per_cta, total, uniform_units, ramp_units;
  int n_pairs;
};

static int spb_of(int block_tokens) { return (block_tokens + kPlanSliceTokens - 1) / kPlanSliceTokens; }

// List positions charged per pair for its fixed costs, in slices: a visit of a pair costs a CTA
// 11-14 us (measured with the phase stamps) against ~0.45 us per 32-token slice of a 256-token
// block; 12..36 all beat 0 on the 28-layer, 32768-token step (157.8 us at 24 against 163.1).
constexpr long long kRampUnits = 24;

static Plan make_plan(long long total_units, int n_pairs, long long uniform_units, int ctas_per_sm) {
  Plan p;
  p.n_pairs = n_pairs;
  p.uniform_units = uniform_units;
  long long slots = (long long)sm_count() * ctas_per_sm;
  long long by_work = total_units / 8 > 1 ? total_units / 8 : 1;   // at least 2 slices per warp
  // a pair cut into more than ~64 parts pays more for the merge of its partial records than the
  // shorter ranges save (single-layer launches: 38 instead of 44 us at 32768 tokens)
  const long long by_pairs = 64ll * n_pairs;
  long long n = slots < by_work ? slots : by_work;
  if (n > by_pairs) n = by_pairs;
  // the ramp charge never exceeds half of an even share of slices
  long long ramp = kRampUnits;
  const long long share = total_units / n;
  if (ramp > share / 2) ramp = share / 2;
  p.ramp_units = ramp;
  p.total = total_units + ramp * n_pairs;
  p.per_cta = (p.total + n - 1) / n;
  p.n_ctas = (int)((p.total + p.per_cta - 1) / p.per_cta);
  return p;
}

extern "C" int64_t inq_decode_units(int32_t n_blocks, int32_t block_tokens) {
  const long long u = (long long)n_blocks * spb_of(block_tokens);
  return u > 0 ? u : 1;
}

extern "C" int64_t inq_decode_workspace_floats(int32_t n_pairs, int64_t total_units) {
  const Plan p = make_plan(total_units > n_pairs ? total_units : n_pairs, n_pairs, 0, 8);
  return ((int64_t)p.n_ctas + n_pairs) * kRecordFloats;
}

extern "C" int inq_decode_attention(const inq_decode_args_t* a, inq_stream_t stream_) {
  if (!a || a->n_seq < 1 || a->kv_heads < 1 || a->q_per_kv < 1 || a->block_tokens < 1) return INQ_ERR_ARGUMENT;
  if (!a->partials || !a->counters || !a->status) return INQ_ERR_ARGUMENT;
  if (a->n_seq > 1 && !a->seqs_device) return INQ_ERR_ARGUMENT;
  if (!a->seqs_device && !a->seq_host) return INQ_ERR_ARGUMENT;
  if (a->dtype != INQ_F16 && a->dtype != INQ_BF16) return INQ_ERR_UNSUPPORTED;
  if (a->layout != 0 && a->layout != 1) return INQ_ERR_ARGUMENT;
  if (!(a->scale > 0.f) || a->n_pad < 0 || a->n_pad > 64) return INQ_ERR_ARGUMENT;
  const int gtiles = (a->q_per_kv + 7) / 8;
  const long long n_pairs = (long long)a->n_seq * a->kv_heads * gtiles;
  if (n_pairs > (1 << 30)) return INQ_ERR_UNSUPPORTED;
  long long uniform = 0, total = 0;
  if (a->pair_starts) {
    if (a->total_units < n_pairs) return INQ_ERR_ARGUMENT;
    total = a->total_units;
  } else {
    const int blocks = a->seqs_device ? a->uniform_blocks : ((const SeqDesc*)a->seq_host)->n_blocks;
    if (blocks < 0) return INQ_ERR_ARGUMENT;
    uniform = inq_decode_units(blocks, a->block_tokens);
    total = uniform * n_pairs;
  }
  const int groups = (a->n_pad + 15) / 16;
  // blocks of at most 16 tokens (16-token pages) take the 16-token-slice kernel: one slice per
  // block either way, so the work list does not depend on the choice
  const int sub = a->block_tokens <= 16 ? 1 : 2;
  typedef void (*kernel_t)(const DecodeParams);
  static const kernel_t kernels[kKernelVariants] = {
      decode_kernel<0, __half, false, 2, false>, decode_kernel<0, __half, true, 2, false>,
      decode_kernel<0, __nv_bfloat16, false, 2, false>, decode_kernel<0, __nv_bfloat16, true, 2, false>,
      decode_kernel<1, __half, false, 2, false>, decode_kernel<1, __half, true, 2, false>,
      decode_kernel<1, __nv_bfloat16, false, 2, false>, decode_kernel<1, __nv_bfloat16, true, 2, false>,
      decode_kernel<0, __half, false, 1, false>, decode_kernel<0, __half, true, 1, false>,
      decode_kernel<0, __nv_bfloat16, false, 1, false>, decode_kernel<0, __nv_bfloat16, true, 1, false>,
      decode_kernel<1, __half, false, 1, false>, decode_kernel<1, __half, true, 1, false>,
      decode_kernel<1, __nv_bfloat16, false, 1, false>, decode_kernel<1, __nv_bfloat16, true, 1, false>,
      // whole slices, at least two per block, one salient group
      decode_kernel<0, __half, true, 2, true>, decode_kernel<0, __nv_bfloat16, true, 2, true>,
      decode_kernel<1, __half, true, 2, true>, decode_kernel<1, __nv_bfloat16, true, 2, true>,
      // the same with the values stored as InQuant packed tensors (table layout)
      decode_kernel<0, __half, true, 2, true, 1>, decode_kernel<0, __nv_bfloat16, true, 2, true, 1>,
      // 4-bit values in 1, 2 or 4 groups
      decode_kernel<0, __half, true, 2, true, 2, 1>, decode_kernel<0, __nv_bfloat16, true, 2, true, 2, 1>,
      decode_kernel<0, __half, true, 2, true, 2, 2>, decode_kernel<0, __nv_bfloat16, true, 2, true, 2, 2>,
      decode_kernel<0, __half, true, 2, true, 2, 4>, decode_kernel<0, __nv_bfloat16, true, 2, true, 2, 4>,
      // 2-bit values in one group of 128 channels, in four groups of 32
      decode_kernel<0, __half, true, 2, true, 0, 1>, decode_kernel<0, __nv_bfloat16, true, 2, true, 0, 1>,
      decode_kernel<0, __half, true, 2, true, 0, 4>, decode_kernel<0, __nv_bfloat16, true, 2, true, 0, 4>};
  const bool fast = a->n_pad == 16 && a->block_tokens % 32 == 0 && a->block_tokens >= 64;
  const int vk = a->value_kind, vg = a->value_groups;
  if (vk < 0 || vk > 2 || (vk == 2 && vg != 1 && vg != 2 && vg != 4) || (vk == 0 && vg != 0 && vg != 1 && vg != 2 && vg != 4))
    return INQ_ERR_ARGUMENT;
  const bool one_group = vk == 0 && (vg == 1 || vg == 4);   // 2-bit values in one group of 128 channels or four of 32
  if (one_group && !(fast && a->layout == 0)) return INQ_ERR_UNSUPPORTED;
  // coded values are served for the whole-slice geometry of the table layout with 16 salient channels
  // on either side; every other combination is inq_decode_generic's
  if (vk && !(fast && a->layout == 0)) return INQ_ERR_UNSUPPORTED;
  if (vk == 1 && !a->seqs_device && ((const SeqDesc*)a->seq_host)->n_blocks > 0 && !((const SeqDesc*)a->seq_host)->value_roles)
    return INQ_ERR_ARGUMENT;
  const int which = one_group ? (vg == 1 ? 28 : 30) + (a->dtype == INQ_F16 ? 0 : 1)
                  : vk == 2 ? 22 + (vg == 1 ? 0 : vg == 2 ? 2 : 4) + (a->dtype == INQ_F16 ? 0 : 1)
                  : vk ? 20 + (a->dtype == INQ_F16 ? 0 : 1)
                  : fast ? 16 + a->layout * 2 + (a->dtype == INQ_F16 ? 0 : 1)
                         : (sub == 1 ? 8 : 0) + a->layout * 4 + (a->dtype == INQ_F16 ? 0 : 2) + (groups > 0 ? 1 : 0);
  const kernel_t kernel = kernels[which];
  const int shared = smem_bytes(groups, sub, vk, vg);
  const int shared_limit = smem_bytes(vk ? 1 : 4, sub, vk, vg);
  const int device = current_device();
  if (device < 0) return INQ_ERR_UNSUPPORTED;   // device ordinals above 63 are not tracked
  int resident = 0;
  {
    std::lock_guard<std::mutex> guard(g_devices_mutex);
    DeviceState& d = g_devices[device];
    if (!d.raised[which]) {
      INQ_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, shared_limit));
      d.raised[which] = true;
    }
    if (!d.per_sm[which][groups]) {
      int n = 0;
      INQ_CUDA_CHECK(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kernel, kThreads, shared));
      d.per_sm[which][groups] = n > 0 ? n : 1;
    }
    resident = d.per_sm[which][groups];
  }
  const Plan plan = make_plan(total, (int)n_pairs, uniform, resident);
  if (((long long)plan.n_ctas + n_pairs) * kRecordFloats > a->partials_floats) return INQ_ERR_CAPACITY;
  DecodeParams P;
  P.seqs = (const SeqDesc*)a->seqs_device;
  if (!a->seqs_device) P.one = *(const SeqDesc*)a->seq_host;
  P.n_seq = a->n_seq;
  P.H = a->kv_heads;
  P.G = a->q_per_kv;
  P.T = a->block_tokens;
  P.n_pad = a->n_pad;
  P.n_ctas = plan.n_ctas;
  P.n_pairs = plan.n_pairs;
  P.per_cta = plan.per_cta;
  P.total_units = plan.total;
  P.uniform_units = plan.uniform_units;
  P.ramp_units = plan.ramp_units;
  P.pair_starts = (const long long*)a->pair_starts;
  P.scale_log2e = a->scale * 1.4426950408889634f;
  P.page_bytes = a->page_bytes;
  P.off_ks = (int)a->page_offsets[0];
  P.off_km = (int)a->page_offsets[1];
  P.off_kp = (int)a->page_offsets[2];
  P.off_vp = (int)a->page_offsets[3];
  P.off_vs = (int)a->page_offsets[4];
  P.off_vo = (int)a->page_offsets[5];
  P.partials = a->partials;
  P.counters = a->counters;
  P.status = a->status;
  P.fused_append = a->fused_append ? 1 : 0;
  P.exchange = (const ExchangeView*)a->exchange_device;
  kernel<<<(unsigned)plan.n_ctas, kThreads, shared, (cudaStream_t)stream_>>>(P);
  INQ_CUDA_CHECK(cudaGetLastError());
  return INQ_OK;
}

// ------------------------------------------------------------------------------------------
// Decode attention for callers that must not allocate.
//
// Serving stacks commonly hand (almost) all device memory to their own page pool at start-up
// and forbid any later cudaMalloc from inside an attention backend: it may fail outright, it
// may fragment the pool, and it is illegal inside a CUDA-graph capture.  A foreign-language
// host (Go, Java, Rust over FFI) that owns device memory through its own allocator is in the
// same position.  For those callers the split-KV partial records and arrival counters live in
// this fixed array instead of caller-provided scratch.  Every process that loads the library
// holds it on every device it uses until exit.
namespace inq {
constexpr int kStaticRecords = 1024;   // (resident CTAs + pairs) of one launch must fit
constexpr int kStaticPairs = 256;      // (sequence, KV head, head tile) pairs of one launch
constexpr size_t kStaticCounterBytes = 2 * kStaticPairs * sizeof(int);   // pair counters, the grid counter, padding
constexpr size_t kStaticBytes = kStaticCounterBytes + (size_t)kStaticRecords * kRecordFloats * sizeof(float);
static __device__ __align__(256) unsigned char g_decode_static_scratch[kStaticBytes];
}  // namespace inq

extern "C" int inq_decode_attention_noalloc(const inq_decode_args_t* a, inq_stream_t stream_) {
  if (!a) return INQ_ERR_ARGUMENT;
  const long long n_pairs = (long long)a->n_seq * a->kv_heads * ((a->q_per_kv + 7) / 8);
  if (a->n_seq < 1 || a->kv_heads < 1 || a->q_per_kv < 1) return INQ_ERR_ARGUMENT;
  if (n_pairs > kStaticPairs) return INQ_ERR_CAPACITY;
  // The array's name is a host-side stand-in, not a device address: resolve it once per device,
  // with that device current, and hand the resolved pointer to the kernel.
  const int device = current_device();
  if (device < 0) return INQ_ERR_UNSUPPORTED;
  void* scratch = nullptr;
  {
    std::lock_guard<std::mutex> guard(g_devices_mutex);
    DeviceState& d = g_devices[device];
    if (!d.static_scratch || d.static_counters_stale) {
      void* ptr = nullptr;
      INQ_CUDA_CHECK(cudaGetSymbolAddress(&ptr, g_decode_static_scratch));
      // The arrival counters must be zero when a launch starts.  Every launch that runs to its end
      // leaves them zero, so they are cleared on the first call on a device and again after a call
      // whose launch was refused by the runtime.  A launch that is cut short on the device (the
      // context is torn down under it) ends the process's use of that context anyway.
      INQ_CUDA_CHECK(cudaMemsetAsync(ptr, 0, kStaticCounterBytes, (cudaStream_t)stream_));
      d.static_scratch = ptr;
      d.static_counters_stale = false;
    }
    scratch = d.static_scratch;
  }
  inq_decode_args_t local = *a;
  local.counters = (int32_t*)scratch;
  local.partials = (float*)((unsigned char*)scratch + kStaticCounterBytes);
  local.partials_floats = (int64_t)kStaticRecords * kRecordFloats;
  const int rc = inq_decode_attention(&local, stream_);   // INQ_ERR_CAPACITY when the launch needs more records
  if (rc == INQ_ERR_CUDA) {
    std::lock_guard<std::mutex> guard(g_devices_mutex);
    g_devices[device].static_counters_stale = true;
  }
  return rc;
}


// ------------------------------------------------------------------------------------------
// Log-sum-exp merge of the un-normalised partial records of several ranks (split-KV across
// GPUs): records [n_parts][n_rows][130] fp32 -> out [n_rows][128].  m is in base-2 units.
namespace inq {
template <typename QT>
__global__ void __launch_bounds__(128) merge_partials_kernel(const float* records, int n_parts, long long n_rows, QT* out) {
  const long long row = blockIdx.x;
  const int c = threadIdx.x;
  float top = kNegBig;
  for (int p = 0; p < n_parts; ++p) top = fmaxf(top, records[((long long)p * n_rows + row) * 130 + 128]);
  float o = 0.f, l = 0.f;
  for (int p = 0; p < n_parts; ++p) {
    const float* rec = records + ((long long)p * n_rows + row) * 130;
    const float w = fast_exp2(rec[128] - top);
    o = fmaf(rec[c], w, o);
    l = fmaf(rec[129], w, l);
  }
  out[row * 128 + c] = from_float<QT>(o / l);
}
}  // namespace inq

extern "C" int inq_merge_partials(const float* records, int32_t n_parts, int64_t n_rows, void* out, int32_t out_dtype,
                                  inq_stream_t stream_) {
  if (!records || !out || n_parts < 1 || n_rows < 1 || n_rows >= (1ll << 31)) return INQ_ERR_ARGUMENT;
  if (out_dtype != INQ_F16 && out_dtype != INQ_BF16) return INQ_ERR_UNSUPPORTED;
  cudaStream_t stream = (cudaStream_t)stream_;
  if (out_dtype == INQ_F16)
    inq::merge_partials_kernel<__half><<<(unsigned)n_rows, 128, 0, stream>>>(records, n_parts, n_rows, (__half*)out);
  else
    inq::merge_partials_kernel<__nv_bfloat16><<<(unsigned)n_rows, 128, 0, stream>>>(records, n_parts, n_rows, (__nv_bfloat16*)out);
  INQ_CUDA_CHECK(cudaGetLastError());
  return INQ_OK;
}

