// Chunked-prefill attention on the 5th-generation tensor cores (tcgen05, accumulators in TMEM).
//
// One CTA owns 256 query tokens of one query head as two tiles of 128 rows (A and B) and walks
// the visible keys and values in tiles of 128 tokens.  Ten warps, three roles:
//   * warps 0-3 / 4-7: softmax of tile A / tile B, one thread per query row.  A thread reads its
//     row of S from tensor memory (tcgen05.ld) once, takes base-2 probabilities against a lazily
//     raised reference maximum (the pass is repeated in the rare case that the maximum has to
//     rise) and writes P in the model dtype back to tensor memory (tcgen05.st) over S.
//   * warp 8 (one lane): issues the contractions.  S = Q K^T (tcgen05.mma 128 x 128 x 128, both
//     operands in shared memory) and O += P V (128 x 128 x 128, P from tensor memory, V as an
//     MN-major shared-memory operand), fp32 accumulators in tensor memory.  The order S_A, S_B,
//     PV_A, S_A', PV_B, S_B', ... keeps the tensor core busy with one tile while the other
//     tile's softmax runs.
//   * warp 9 (one lane): TMA (cp.async.bulk.tensor, 128-byte swizzle, no multicast) for Q once and
//     for the double-buffered K and V tiles.
// All hand-overs are mbarriers; every wait is bounded and a wait that gives up raises an abort
// flag that ends the other loops.  One CTA per SM (tensor-memory kernels are scheduled that way),
// 192 KB of shared memory, all 512 TMEM columns.  Keys and values are dense tensors in the model
// dtype: the dequantised packed history followed by the chunk's own tokens; query i sees
// positions <= history + i.
//
// Shared-memory operand tiles hold 128 rows of 128 2-byte elements as two slabs of 64 columns;
// inside a slab a row is 128 bytes and its 16-byte chunks are XOR-swizzled with the row index
// modulo 8 (the 128-byte swizzle of the tensor-core descriptors).
#include <cuda.h>

#include <algorithm>
#include <type_traits>

#include "common.cuh"

namespace inq {

constexpr int kPfThreads = 320;              // 8 softmax warps, the MMA warp, the TMA warp
constexpr int kPfTile = 128;                 // query rows per tile, KV tokens per tile, head dimension
constexpr int kPfRows = 2 * kPfTile;         // query rows per CTA (tiles A and B)
constexpr int kPfSlab = kPfTile * 128;       // 128 rows x 128 bytes
constexpr int kPfTileBytes = 2 * kPfSlab;    // one operand tile: two slabs (64-column halves)
constexpr int kPfStages = 2;                 // K and V tiles in flight
constexpr int kPfTiles = (2 + 2 * kPfStages) * kPfTileBytes;   // Q x2, K and V stages
constexpr int kPfSmem = kPfTiles + 160;      // then the TMEM base address, the abort flag and 11 mbarriers
constexpr int kPfTmemCols = 512;             // S_A 0..127, S_B 128..255 (P over their first 64), O_A 256..383, O_B 384..511
constexpr float kPfNegBig = -1.0e30f;
constexpr float kPfSlack = 8.f;              // the reference maximum may lag the true one by 2^8 (P stays below 256)
constexpr int kPfSpinLimit = 1 << 22;
constexpr int kPfMaxSplits = 8;              // KV segments per item at most

struct PrefillParams {
  const void *q, *k, *v;
  void* out;
  long long q_sh, q_st, k_sh, k_st, v_sh, v_st, o_sh, o_st;   // strides in elements
  int q_heads, kv_heads, q_tokens, kv_tokens, n_qpairs;
  int splits;         // KV segments per (query pair, head) item; > 1 writes partial records
  float* records;     // [items][splits][256 rows][130]: unnormalised O, reference maximum, sum
  float scale_log2e;
  int* status;
};

__device__ __forceinline__ unsigned pf_smem(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }

// 64-bit shared-memory matrix descriptor, 128-byte swizzle: start address, leading and stride
// byte offsets in 16-byte units, descriptor version 1, layout type 2.
__device__ __forceinline__ unsigned long long pf_desc(unsigned saddr, unsigned lbo_bytes, unsigned sbo_bytes) {
  unsigned long long d = 0;
  d |= (unsigned long long)((saddr & 0x3FFFFu) >> 4);
  d |= (unsigned long long)(lbo_bytes >> 4) << 16;
  d |= (unsigned long long)(sbo_bytes >> 4) << 32;
  d |= 1ull << 46;
  d |= 2ull << 61;
  return d;
}

__device__ __forceinline__ void pf_mma(unsigned tmem_d, unsigned long long da, unsigned long long db, unsigned idesc,
                                       unsigned accumulate) {
  asm volatile("{ .reg .pred p; setp.ne.b32 p, %4, 0; tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p; }"
               ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void pf_mma_ta(unsigned tmem_d, unsigned tmem_a, unsigned long long db, unsigned idesc,
                                          unsigned accumulate) {
  asm volatile("{ .reg .pred p; setp.ne.b32 p, %4, 0; tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p; }"
               ::"r"(tmem_d), "r"(tmem_a), "l"(db), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void pf_commit(unsigned mbar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(mbar) : "memory");
}
// Bounded wait; gives up early when another role has raised the abort flag.
__device__ __forceinline__ bool pf_wait(unsigned mbar, unsigned parity, volatile int* abort_flag) {
  for (int it = 0; it < kPfSpinLimit; ++it) {
    unsigned done;
    asm volatile("{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
                 : "=r"(done) : "r"(mbar), "r"(parity) : "memory");
    if (done) return true;
    if ((it & 255) == 255 && *abort_flag) return false;
  }
  *abort_flag = 1;
  return false;
}
__device__ __forceinline__ void pf_arrive(unsigned mbar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(mbar) : "memory");
}
__device__ __forceinline__ void pf_tmem_ld32(unsigned taddr, unsigned (&v)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,"
      "%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
        "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]),
        "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]),
        "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
      : "r"(taddr) : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void pf_tmem_st32(unsigned taddr, const unsigned (&v)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,"
      "%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
      ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]),
        "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]), "r"(v[16]), "r"(v[17]),
        "r"(v[18]), "r"(v[19]), "r"(v[20]), "r"(v[21]), "r"(v[22]), "r"(v[23]), "r"(v[24]), "r"(v[25]), "r"(v[26]),
        "r"(v[27]), "r"(v[28]), "r"(v[29]), "r"(v[30]), "r"(v[31])
      : "memory");
}
__device__ __forceinline__ float pf_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
template <typename QT>
__device__ __forceinline__ unsigned pf_pack2(float lo, float hi) {
  if (std::is_same<QT, __half>::value) {
    __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<unsigned*>(&h);
  }
  __nv_bfloat162 b = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<unsigned*>(&b);
}

// One TMA box: 64 columns (128 bytes) x `rows` rows of head `z`, starting at column x and row y, into
// a swizzled slab; rows beyond the tensor are zero-filled by the hardware.
__device__ __forceinline__ void pf_tma(unsigned dst, const CUtensorMap* map, int x, int y, int z, unsigned mbar) {
  asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
               ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(z), "r"(mbar) : "memory");
}
__device__ __forceinline__ void pf_expect(unsigned mbar, unsigned bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(mbar), "r"(bytes) : "memory");
}

template <typename QT>
__global__ void __launch_bounds__(kPfThreads, 1) prefill_kernel(const PrefillParams P, const __grid_constant__ CUtensorMap map_q,
                                                                const __grid_constant__ CUtensorMap map_k,
                                                                const __grid_constant__ CUtensorMap map_v) {
  // no static shared memory: the dynamic region starts the CTA's window, 1024-byte aligned as the
  // 128-byte swizzle needs (checked below)
  extern __shared__ __align__(1024) unsigned char pf_raw[];
  const unsigned smem0 = pf_smem(pf_raw);
  const unsigned sQ = smem0;                                  // tile A, then tile B
  const unsigned sKb = smem0 + 2 * kPfTileBytes;              // K stages
  const unsigned sVb = sKb + kPfStages * kPfTileBytes;        // V stages
  unsigned* const tmem_base_p = (unsigned*)(pf_raw + kPfTiles);
  volatile int* const abort_flag = (volatile int*)(pf_raw + kPfTiles + 4);
  const unsigned bars = smem0 + kPfTiles + 16;
  const unsigned bar_q = bars, bar_k = bars + 8 /* per stage */, bar_v = bar_k + 8 * kPfStages /* per stage */;
  const unsigned bar_s = bar_v + 8 * kPfStages /* A, B */, bar_p = bar_s + 16 /* A, B */, bar_o = bar_p + 16 /* A, B */;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (smem0 & 1023u) {
    if (tid == 0) atomicOr(P.status, INQ_STATUS_BAD_INDEX);
    return;
  }

  // An item is (256 query rows, query head); late query rows see the most keys and are scheduled
  // first.  With P.splits > 1 every item is cut into that many KV segments, one CTA each, so that
  // the grid fills the SMs evenly; the segments' partial results are merged by a second kernel.
  const int item = (int)(blockIdx.x / P.splits), seg = (int)(blockIdx.x % P.splits);
  const int qp = P.n_qpairs - 1 - item / P.q_heads;
  const int head = item % P.q_heads;
  const int kvh = head / (P.q_heads / P.kv_heads);
  const int q0 = qp * kPfRows;
  const int hist = P.kv_tokens - P.q_tokens;
  // tiles each query tile needs: A ends at its last row's diagonal, B 128 tokens later; this CTA
  // walks tiles [t_lo, t_hi) and n_a / n_b count the tiles of its segment
  const int all_a = (min(P.kv_tokens, hist + q0 + kPfTile) + kPfTile - 1) / kPfTile;
  const int all_b = (min(P.kv_tokens, hist + q0 + kPfRows) + kPfTile - 1) / kPfTile;
  const int t_lo = (int)((long long)all_b * seg / P.splits), t_hi = (int)((long long)all_b * (seg + 1) / P.splits);
  const int n_b = t_hi - t_lo;
  const int n_a = max(0, min(all_a, t_hi) - t_lo);

  if (tid == 0) {
    *abort_flag = 0;
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(bar_q) : "memory");
#pragma unroll
    for (int i = 0; i < kPfStages; ++i) {
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(bar_k + 8 * i) : "memory");
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(bar_v + 8 * i) : "memory");
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(bar_s + 8 * i) : "memory");
      asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar_p + 8 * i), "r"(kPfTile) : "memory");
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(bar_o + 8 * i) : "memory");
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 8) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                 ::"r"(pf_smem(tmem_base_p)), "r"(kPfTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const unsigned tmem = *tmem_base_p;

  if (warp == 9) {
    // ================================================================ TMA warp
    if (lane == 0 && n_b > 0) {
      auto request_k = [&](int t) {
        const unsigned bar = bar_k + 8 * (t % kPfStages), dst = sKb + (t % kPfStages) * kPfTileBytes;
        pf_expect(bar, kPfTileBytes);
        pf_tma(dst, &map_k, 0, (t_lo + t) * kPfTile, kvh, bar);
        pf_tma(dst + kPfSlab, &map_k, 64, (t_lo + t) * kPfTile, kvh, bar);
      };
      auto request_v = [&](int t) {
        const unsigned bar = bar_v + 8 * (t % kPfStages), dst = sVb + (t % kPfStages) * kPfTileBytes;
        pf_expect(bar, kPfTileBytes);
        pf_tma(dst, &map_v, 0, (t_lo + t) * kPfTile, kvh, bar);
        pf_tma(dst + kPfSlab, &map_v, 64, (t_lo + t) * kPfTile, kvh, bar);
      };
      pf_expect(bar_q, 2 * kPfTileBytes);
#pragma unroll
      for (int x = 0; x < 2; ++x) {
        pf_tma(sQ + x * kPfTileBytes, &map_q, 0, q0 + x * kPfTile, head, bar_q);
        pf_tma(sQ + x * kPfTileBytes + kPfSlab, &map_q, 64, q0 + x * kPfTile, head, bar_q);
      }
      for (int t = 0; t < kPfStages && t < n_b; ++t) {
        request_k(t);
        request_v(t);
      }
      for (int t = 0; t + kPfStages < n_b; ++t) {
        // K(t) is free once both score contractions of tile t are done, V(t) once both output
        // contractions are (the commits are ordered, so tile B's barrier covers tile A's)
        if (!pf_wait(bar_s + 8, (unsigned)t & 1u, abort_flag)) break;
        request_k(t + kPfStages);
        if (!pf_wait(bar_o + 8, (unsigned)t & 1u, abort_flag)) break;
        request_v(t + kPfStages);
      }
    }
  } else if (warp == 8) {
    // ================================================================ MMA warp
    if (lane == 0 && n_b > 0) {
      // instruction descriptors: fp32 accumulate, A/B in the model dtype, M = N = 128; the value
      // tile is an MN-major B operand (tokens are its K dimension, stored row by row)
      const unsigned fmt = std::is_same<QT, __half>::value ? 0u : 1u;
      const unsigned idesc_s = (1u << 4) | (fmt << 7) | (fmt << 10) | ((128u >> 3) << 17) | ((128u >> 4) << 24);
      const unsigned idesc_o = idesc_s | (1u << 16);
      auto issue_s = [&](int x, int t) {      // S_x = Q_x K(t)^T
        const unsigned q = sQ + x * kPfTileBytes, k = sKb + (t % kPfStages) * kPfTileBytes;
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          const unsigned off = (kk >> 2) * kPfSlab + (kk & 3) * 32;
          pf_mma(tmem + x * kPfTile, pf_desc(q + off, 16, 1024), pf_desc(k + off, 16, 1024), idesc_s, kk > 0);
        }
        pf_commit(bar_s + 8 * x);
      };
      auto issue_o = [&](int x, int t) {      // O_x += P_x V(t): 16 tokens per step = 8 columns of packed P
        const unsigned v = sVb + (t % kPfStages) * kPfTileBytes;
#pragma unroll
        for (int kk = 0; kk < 8; ++kk)
          pf_mma_ta(tmem + 2 * kPfTile + x * kPfTile, tmem + x * kPfTile + kk * 8, pf_desc(v + kk * 2048, kPfSlab, 1024), idesc_o,
                    (t > 0 || kk > 0) ? 1u : 0u);
        pf_commit(bar_o + 8 * x);
      };
      bool ok = pf_wait(bar_q, 0, abort_flag) && pf_wait(bar_k, 0, abort_flag);
      if (ok) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if (n_a > 0) issue_s(0, 0);
        issue_s(1, 0);
      }
      for (int t = 0; ok && t < n_b; ++t) {
        const bool a_live = t < n_a;
        if (a_live) ok = ok && pf_wait(bar_p, (unsigned)t & 1u, abort_flag);       // P_A(t) written, S_A(t) read
        ok = ok && pf_wait(bar_v + 8 * (t % kPfStages), (unsigned)(t / kPfStages) & 1u, abort_flag);
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if (a_live) issue_o(0, t);
        if (t + 1 < n_b) {
          ok = pf_wait(bar_k + 8 * ((t + 1) % kPfStages), (unsigned)((t + 1) / kPfStages) & 1u, abort_flag);
          if (!ok) break;
          if (t + 1 < n_a) issue_s(0, t + 1);
        }
        ok = pf_wait(bar_p + 8, (unsigned)t & 1u, abort_flag);                     // P_B(t) written, S_B(t) read
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        issue_o(1, t);
        if (t + 1 < n_b) issue_s(1, t + 1);
      }
    }
  } else {
    // ================================================================ softmax warps
    const int x = warp >> 2;                       // 0: tile A, 1: tile B
    const int row = tid & (kPfTile - 1);           // query row inside the tile = TMEM lane
    const int n_x = x ? n_b : n_a;
    const int q_row = q0 + x * kPfTile + row;
    const int q_pos = hist + q_row;                // keys at positions <= q_pos are visible
    const int diag0 = hist + q0 + x * kPfTile;     // first row's diagonal: tiles reaching beyond it need masks
    const unsigned lane_field = (unsigned)((warp & 3) * 32) << 16;
    const unsigned tS = tmem + lane_field + x * kPfTile, tO = tmem + lane_field + 2 * kPfTile + x * kPfTile;
    const unsigned my_s = bar_s + 8 * x, my_p = bar_p + 8 * x, my_o = bar_o + 8 * x;
    float m_ref = kPfNegBig, l_sum = 0.f;
    bool ok = true;

    for (int t = 0; t < n_x; ++t) {
      const int kv0 = (t_lo + t) * kPfTile;
      // S(t) is complete; the contractions run in issue order, so PV(t-1) is complete as well:
      // the columns of P may be overwritten by S and O may be rescaled
      if (!pf_wait(my_s, (unsigned)t & 1u, abort_flag)) { ok = false; break; }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const bool masked = kv0 + kPfTile - 1 > diag0;
      // ---- one pass over S: probabilities against the running reference maximum are packed
      //      into registers while the row maximum is tracked; P is stored over S only afterwards,
      //      so the rare case of a maximum that has to be raised can simply take the pass again
      unsigned packed[64];
      float smax, l_tile;
      auto pass = [&](auto masked_tag) {
        constexpr bool kMasked = decltype(masked_tag)::value;
        smax = kPfNegBig;
        l_tile = 0.f;
#pragma unroll
        for (int c0 = 0; c0 < kPfTile; c0 += 32) {
          unsigned v[32];
          pf_tmem_ld32(tS + c0, v);
#pragma unroll
          for (int c = 0; c < 32; c += 2) {
            const float s0 = __uint_as_float(v[c]), s1 = __uint_as_float(v[c + 1]);
            float e0 = pf_exp2(fmaf(s0, P.scale_log2e, -m_ref));
            float e1 = pf_exp2(fmaf(s1, P.scale_log2e, -m_ref));
            if (kMasked) {
              const bool vis0 = kv0 + c0 + c <= q_pos, vis1 = kv0 + c0 + c + 1 <= q_pos;
              if (vis0) smax = fmaxf(smax, s0); else e0 = 0.f;
              if (vis1) smax = fmaxf(smax, s1); else e1 = 0.f;
            } else {
              smax = fmaxf(smax, fmaxf(s0, s1));
            }
            l_tile += e0 + e1;
            packed[(c0 + c) >> 1] = pf_pack2<QT>(e0, e1);
          }
        }
      };
      if (masked) pass(std::true_type{}); else pass(std::false_type{});
      const bool raise = smax * P.scale_log2e > m_ref + kPfSlack;
      if (__any_sync(0xffffffffu, raise)) {
        // rare after the first tile: bring the running sum and the output accumulator to the new
        // reference maximum, then take the probabilities again
        const float m_new = raise ? smax * P.scale_log2e : m_ref;
        const float factor = pf_exp2(m_ref - m_new);
        l_sum *= factor;
        m_ref = m_new;
        if (t > 0) {
#pragma unroll 1
          for (int c0 = 0; c0 < kPfTile; c0 += 32) {
            unsigned v[32];
            pf_tmem_ld32(tO + c0, v);
#pragma unroll
            for (int c = 0; c < 32; ++c) v[c] = __float_as_uint(__uint_as_float(v[c]) * factor);
            pf_tmem_st32(tO + c0, v);
          }
        }
        if (masked) pass(std::true_type{}); else pass(std::false_type{});
      }
      l_sum += l_tile;
      {
        unsigned lo[32], hi[32];
#pragma unroll
        for (int c = 0; c < 32; ++c) {
          lo[c] = packed[c];
          hi[c] = packed[32 + c];
        }
        pf_tmem_st32(tS, lo);
        pf_tmem_st32(tS + 32, hi);
      }
      // P is in tensor memory, S has been read: hand both to the MMA warp
      asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      pf_arrive(my_p);
    }
    if (n_x > 0) ok = ok && pf_wait(my_o, (unsigned)(n_x - 1) & 1u, abort_flag);
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");

    if (P.splits == 1) {
      // ---- normalise and store this thread's row
      const float inv = 1.f / l_sum;
      const bool live = ok && q_row < P.q_tokens;
      QT* orow = (QT*)P.out + (long long)head * P.o_sh + (long long)q_row * P.o_st;
#pragma unroll 1
      for (int c0 = 0; c0 < kPfTile; c0 += 32) {
        unsigned v[32];
        pf_tmem_ld32(tO + c0, v);
        if (live) {
#pragma unroll
          for (int q4 = 0; q4 < 4; ++q4) {
            uint4 w;
            w.x = pf_pack2<QT>(__uint_as_float(v[8 * q4 + 0]) * inv, __uint_as_float(v[8 * q4 + 1]) * inv);
            w.y = pf_pack2<QT>(__uint_as_float(v[8 * q4 + 2]) * inv, __uint_as_float(v[8 * q4 + 3]) * inv);
            w.z = pf_pack2<QT>(__uint_as_float(v[8 * q4 + 4]) * inv, __uint_as_float(v[8 * q4 + 5]) * inv);
            w.w = pf_pack2<QT>(__uint_as_float(v[8 * q4 + 6]) * inv, __uint_as_float(v[8 * q4 + 7]) * inv);
            *(uint4*)(orow + c0 + 8 * q4) = w;
          }
        }
      }
    } else {
      // ---- partial record of this row: unnormalised output, reference maximum, sum
      float* rec = P.records + (((long long)item * P.splits + seg) * kPfRows + x * kPfTile + row) * 130;
      const bool have = ok && n_x > 0;
#pragma unroll 1
      for (int c0 = 0; c0 < kPfTile; c0 += 32) {
        unsigned v[32];
        if (n_x > 0) {
          pf_tmem_ld32(tO + c0, v);
        }
#pragma unroll
        for (int q4 = 0; q4 < 8; ++q4) {
          float4 w = make_float4(0.f, 0.f, 0.f, 0.f);
          if (have) w = make_float4(__uint_as_float(v[4 * q4]), __uint_as_float(v[4 * q4 + 1]), __uint_as_float(v[4 * q4 + 2]),
                                    __uint_as_float(v[4 * q4 + 3]));
          *(float2*)(rec + c0 + 4 * q4) = make_float2(w.x, w.y);
          *(float2*)(rec + c0 + 4 * q4 + 2) = make_float2(w.z, w.w);
        }
      }
      rec[128] = have ? m_ref : kPfNegBig;
      rec[129] = have ? l_sum : 0.f;
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (tid == 0 && *abort_flag) atomicOr(P.status, INQ_STATUS_WAIT_TIMEOUT);
  if (warp == 8)
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kPfTmemCols) : "memory");
}

// Merges the KV segments of every item: out = sum_s O_s 2^(m_s - m) / sum_s l_s 2^(m_s - m).
// One block per (item, 8 rows): a warp owns a row, a lane four channels, and the loads of all
// segments are issued before the first is used.
constexpr int kPfMergeRows = 8;
template <typename QT>
__global__ void __launch_bounds__(kPfMergeRows * 32) prefill_merge_kernel(const PrefillParams P) {
  const int item = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int qp = P.n_qpairs - 1 - item / P.q_heads, head = item % P.q_heads;
  const int row = blockIdx.y * kPfMergeRows + warp, q_row = qp * kPfRows + row;
  if (q_row >= P.q_tokens) return;
  const float* base = P.records + ((long long)item * P.splits * kPfRows + row) * 130;   // rows are 520 B apart: 8-byte aligned
  float2 ml[kPfMaxSplits], va[kPfMaxSplits], vb[kPfMaxSplits];
#pragma unroll
  for (int sgm = 0; sgm < kPfMaxSplits; ++sgm) {
    if (sgm < P.splits) {
      const float2* rec = (const float2*)(base + (long long)sgm * kPfRows * 130);
      ml[sgm] = __ldcg(rec + 64);
      va[sgm] = __ldcg(rec + 2 * lane);
      vb[sgm] = __ldcg(rec + 2 * lane + 1);
    }
  }
  float top = kPfNegBig;
#pragma unroll
  for (int sgm = 0; sgm < kPfMaxSplits; ++sgm)
    if (sgm < P.splits) top = fmaxf(top, ml[sgm].x);
  float o0 = 0.f, o1 = 0.f, o2 = 0.f, o3 = 0.f, l = 0.f;
#pragma unroll
  for (int sgm = 0; sgm < kPfMaxSplits; ++sgm) {
    if (sgm < P.splits) {
      const float w = pf_exp2(ml[sgm].x - top);
      o0 = fmaf(va[sgm].x, w, o0);
      o1 = fmaf(va[sgm].y, w, o1);
      o2 = fmaf(vb[sgm].x, w, o2);
      o3 = fmaf(vb[sgm].y, w, o3);
      l = fmaf(ml[sgm].y, w, l);
    }
  }
  QT* out = (QT*)P.out + (long long)head * P.o_sh + (long long)q_row * P.o_st + 4 * lane;
  out[0] = from_float<QT>(o0 / l);
  out[1] = from_float<QT>(o1 / l);
  out[2] = from_float<QT>(o2 / l);
  out[3] = from_float<QT>(o3 / l);
}

}  // namespace inq

using namespace inq;

namespace {
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn encode_tiled() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult result;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &result) == cudaSuccess &&
        result == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)p;
  }
  return fn;
}
// [heads][tokens][128] tensor of 2-byte elements, boxes of 64 columns x `box_rows` rows, 128-byte swizzle
bool make_map(CUtensorMap* map, const void* base, int dtype, long long tokens, long long heads, long long stride_t,
              long long stride_h, int box_rows) {
  EncodeTiledFn fn = encode_tiled();
  if (!fn) return false;
  if (heads == 1) stride_h = tokens * stride_t;   // unused, but must be a valid stride
  const cuuint64_t dims[3] = {128, (cuuint64_t)tokens, (cuuint64_t)heads};
  const cuuint64_t strides[2] = {(cuuint64_t)stride_t * 2, (cuuint64_t)stride_h * 2};
  const cuuint32_t box[3] = {64, (cuuint32_t)box_rows, 1};
  const cuuint32_t elem[3] = {1, 1, 1};
  return fn(map, dtype == INQ_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, (void*)base, dims,
            strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}
}  // namespace


// Cuts only pay while the items are few compared with the SMs: at most 2048 segments in all, which
// also bounds the scratch at 2048 partial records (272 MB).
static int max_splits(long long items) {
  return (int)std::max<long long>(1, std::min<long long>(kPfMaxSplits, 2048 / std::max<long long>(items, 1)));
}

extern "C" int64_t inq_prefill_workspace_bytes(int32_t q_heads, int32_t q_tokens) {
  const long long items = (long long)((q_tokens + kPfRows - 1) / kPfRows) * q_heads;
  const int sp = max_splits(items);
  return sp > 1 ? items * sp * kPfRows * 130 * (long long)sizeof(float) : 0;
}

extern "C" int inq_prefill_attention(const inq_prefill_args_t* a, inq_stream_t stream_) {
  if (!a || !a->q || !a->k || !a->v || !a->out || !a->status) return INQ_ERR_ARGUMENT;
  if (a->q_heads < 1 || a->kv_heads < 1 || a->q_heads % a->kv_heads) return INQ_ERR_ARGUMENT;
  if (a->q_tokens < 1 || a->kv_tokens < a->q_tokens || !(a->scale > 0.f)) return INQ_ERR_ARGUMENT;
  if (a->dtype != INQ_F16 && a->dtype != INQ_BF16) return INQ_ERR_UNSUPPORTED;
  // rows are read and written as 16-byte vectors
  if ((a->q_stride_t | a->k_stride_t | a->v_stride_t | a->o_stride_t | a->q_stride_h | a->k_stride_h | a->v_stride_h |
       a->o_stride_h) & 7)
    return INQ_ERR_ARGUMENT;
  if (((uintptr_t)a->q | (uintptr_t)a->k | (uintptr_t)a->v | (uintptr_t)a->out) & 15) return INQ_ERR_ARGUMENT;
  PrefillParams P;
  P.q = a->q; P.k = a->k; P.v = a->v; P.out = a->out;
  P.q_sh = a->q_stride_h; P.q_st = a->q_stride_t; P.k_sh = a->k_stride_h; P.k_st = a->k_stride_t;
  P.v_sh = a->v_stride_h; P.v_st = a->v_stride_t; P.o_sh = a->o_stride_h; P.o_st = a->o_stride_t;
  P.q_heads = a->q_heads; P.kv_heads = a->kv_heads; P.q_tokens = a->q_tokens; P.kv_tokens = a->kv_tokens;
  P.n_qpairs = (a->q_tokens + kPfRows - 1) / kPfRows;
  P.splits = 1;
  P.records = (float*)a->workspace;
  {
    // cut every item into `splits` KV segments when that fills the SMs more evenly: rounds of
    // CTAs over the SMs, each round as long as one segment, a few per cent of overhead per cut
    int n_sm = 0, device = 0;   // asked per call: the answer belongs to the current device
    INQ_CUDA_CHECK(cudaGetDevice(&device));
    INQ_CUDA_CHECK(cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, device));
    const long long items = (long long)P.n_qpairs * a->q_heads;
    const int lightest = (int)((std::min<long long>(a->kv_tokens, (long long)a->kv_tokens - a->q_tokens + kPfRows) + kPfTile - 1) / kPfTile);
    // cost of a cut into sp segments, in KV-tile times: rounds of CTAs over the SMs, each as long
    // as one segment plus, when cut, the fixed price of a segment (pipeline fill, writing and
    // merging a 133 KB partial record), measured at about six tile times
    const double tiles = ((double)a->kv_tokens - 0.5 * a->q_tokens) / kPfTile;
    double best = 1e30;
    for (int sp = 1; sp <= max_splits(items); ++sp) {
      if (sp > 1 && (lightest / sp < 2 || !a->workspace ||
                     a->workspace_bytes < (long long)items * sp * kPfRows * 130 * (long long)sizeof(float)))
        break;
      const double rounds = (double)((items * sp + n_sm - 1) / n_sm);
      const double cost = rounds * (tiles / sp + (sp > 1 ? 6.0 : 0.0));
      if (cost < best - 1e-9) {
        best = cost;
        P.splits = sp;
      }
    }
  }
  P.scale_log2e = a->scale * 1.4426950408889634f;
  P.status = a->status;
  const long long ctas = (long long)P.n_qpairs * P.q_heads * P.splits;
  if (ctas > 0x7fffffffLL) return INQ_ERR_CAPACITY;
  cudaStream_t stream = (cudaStream_t)stream_;
  if (a->q_stride_h <= 0 || a->k_stride_h <= 0 || a->v_stride_h <= 0 || a->q_stride_t < 128 || a->k_stride_t < 128 ||
      a->v_stride_t < 128)
    return INQ_ERR_ARGUMENT;
  CUtensorMap map_q, map_k, map_v;
  if (!make_map(&map_q, a->q, a->dtype, a->q_tokens, a->q_heads, a->q_stride_t, a->q_stride_h, kPfTile) ||
      !make_map(&map_k, a->k, a->dtype, a->kv_tokens, a->kv_heads, a->k_stride_t, a->k_stride_h, kPfTile) ||
      !make_map(&map_v, a->v, a->dtype, a->kv_tokens, a->kv_heads, a->v_stride_t, a->v_stride_h, kPfTile))
    return INQ_ERR_ARGUMENT;
  if (a->dtype == INQ_F16) {
    INQ_CUDA_CHECK(cudaFuncSetAttribute(prefill_kernel<__half>, cudaFuncAttributeMaxDynamicSharedMemorySize, kPfSmem));
    prefill_kernel<__half><<<(unsigned)ctas, kPfThreads, kPfSmem, stream>>>(P, map_q, map_k, map_v);
    if (P.splits > 1) prefill_merge_kernel<__half><<<dim3((unsigned)(ctas / P.splits), kPfRows / kPfMergeRows), kPfMergeRows * 32, 0, stream>>>(P);
  } else {
    INQ_CUDA_CHECK(cudaFuncSetAttribute(prefill_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, kPfSmem));
    prefill_kernel<__nv_bfloat16><<<(unsigned)ctas, kPfThreads, kPfSmem, stream>>>(P, map_q, map_k, map_v);
    if (P.splits > 1) prefill_merge_kernel<__nv_bfloat16><<<dim3((unsigned)(ctas / P.splits), kPfRows / kPfMergeRows), kPfMergeRows * 32, 0, stream>>>(P);
  }
  INQ_CUDA_CHECK(cudaGetLastError());
  return INQ_OK;
}
