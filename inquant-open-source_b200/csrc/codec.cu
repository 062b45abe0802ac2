// K4 key encoder (sampled statistics + donor selection + mixed 4/8-bit packing), V2/V4
// group-wise value encoder, their exact inverses and the role-map builder.
//
// Compile this translation unit with -fmad=false: the packed bytes must equal the
// reference's bit for bit, and the reference performs separate IEEE multiplies, adds and
// divisions.  The only fused operations are the explicit fma() calls of the division-by-
// integer below, which is proven to return the correctly rounded quotient.
#include <algorithm>

#include "common.cuh"

namespace inq {

constexpr int kMaxChannels = 1024;
constexpr int kMaxWords = kMaxChannels / 32;
constexpr int kRcpTable = 512;  // tokens per row for which 1/(t+1) is tabulated in shared memory

// ------------------------------------------------------------------------------------------
// Sampled statistics in the summation order of the reference's CPU reduction: samples are
// added one by one into a level-0 accumulator that is folded into level 1 every `step`
// samples (level 1 into level 2 every step^2, ...), a remainder shorter than `step` stays in
// level 0, and the levels are added lowest first at the end.
struct CascadePair {
  float abs_acc[4], sum_acc[4];
  int i, full_end, mask, level_power;
  __device__ void init(int n) {
#pragma unroll
    for (int k = 0; k < 4; ++k) abs_acc[k] = sum_acc[k] = 0.f;
    int ceil_log2 = n <= 1 ? 0 : 32 - __clz(n - 1);
    level_power = max(4, ceil_log2 / 4);
    int step = 1 << level_power;
    mask = step - 1;
    full_end = (n / step) * step;
    i = 0;
  }
  __device__ void add(float v) {
    abs_acc[0] = abs_acc[0] + fabsf(v);
    sum_acc[0] = sum_acc[0] + v;
    ++i;
    if (i <= full_end && (i & mask) == 0) {
#pragma unroll
      for (int level = 1; level < 4; ++level) {
        abs_acc[level] = abs_acc[level] + abs_acc[level - 1];
        sum_acc[level] = sum_acc[level] + sum_acc[level - 1];
        abs_acc[level - 1] = 0.f;
        sum_acc[level - 1] = 0.f;
        if (i & (mask << (level * level_power))) break;
      }
    }
  }
  __device__ void finish(float& abs_total, float& sum_total) {
#pragma unroll
    for (int level = 1; level < 4; ++level) {
      abs_acc[0] = abs_acc[0] + abs_acc[level];
      sum_acc[0] = sum_acc[0] + sum_acc[level];
    }
    abs_total = abs_acc[0];
    sum_total = sum_acc[0];
  }
};

// d / n for a small positive integer n, given y = RN(1/n): one multiply and two fused
// corrections return the correctly rounded IEEE quotient (Markstein's theorem).
__device__ __forceinline__ double divide_by_count(double d, double n, double y) {
  double q0 = d * y;
  double r = fma(-q0, n, d);
  return fma(r, y, q0);
}

struct ChannelStats {
  float saliency, sampled_mean, donor_error, absmax;
  bool finite;
};

// One thread walks one channel over all tokens of a row.
template <typename T>
__device__ ChannelStats channel_statistics(const T* column, long long s_token, int tokens, int sample_stride,
                                           bool want_error, const double* rcp_table) {
  ChannelStats out;
  CascadePair cascade;
  int samples = (tokens + sample_stride - 1) / sample_stride;
  cascade.init(samples);
  float absmax = 0.f;
  bool finite = true;
  double mean = 0.0, m2 = 0.0;
  int next_sample = 0;
  constexpr int kUnroll = 8;
  for (int base = 0; base < tokens; base += kUnroll) {
    float v[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      int t = base + u;
      v[u] = t < tokens ? to_float<T>(column[(long long)t * s_token]) : 0.f;
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      int t = base + u;
      if (t < tokens) {
        float x = v[u];
        finite = finite && finite_f32(x);
        absmax = fmaxf(absmax, fabsf(x));
        if (t == next_sample) {
          cascade.add(x);
          next_sample += sample_stride;
        }
        if (want_error) {
          // Welford's update in float64, sequential over tokens (torch CPU var_mean).
          double xd = (double)x;
          double delta = xd - mean;
          double q = rcp_table ? divide_by_count(delta, (double)(t + 1), rcp_table[t]) : delta / (double)(t + 1);
          mean = mean + q;
          m2 = m2 + delta * (xd - mean);
        }
      }
    }
  }
  float abs_total, sum_total;
  cascade.finish(abs_total, sum_total);
  out.saliency = abs_total / (float)samples;
  out.sampled_mean = sum_total / (float)samples;
  out.absmax = absmax;
  out.finite = finite;
  out.donor_error = 0.f;
  if (want_error) {
    float variance = (float)(m2 / (double)tokens);
    float diff = (float)mean - out.sampled_mean;
    out.donor_error = variance + diff * diff;
  }
  return out;
}

// ------------------------------------------------------------------------------------------
// Donor selection.  Called by every thread of a CTA whose blockDim.x >= channels.
// Shared inputs: saliency[C], error[C] (if use_error).  Shared scratch: rank_key[C] (u32),
// sel_mask / avail_mask [NW words].  Outputs in shared memory: sources[count] ascending,
// donors[count].
template <int NW>
__device__ int highest_below(const unsigned (&mask)[NW], int pos) {  // largest set index < pos, or -1
  int w = pos >> 5;
  if (w < NW) {
    unsigned m = (pos & 31) ? (mask[w] & ((1u << (pos & 31)) - 1u)) : 0u;
    if (m) return (w << 5) + 31 - __clz(m);
  }
  for (int k = min(w, NW) - 1; k >= 0; --k)
    if (mask[k]) return (k << 5) + 31 - __clz(mask[k]);
  return -1;
}
template <int NW>
__device__ int lowest_above(const unsigned (&mask)[NW], int pos, int limit) {  // smallest set index > pos, or limit
  int start = pos + 1;
  int w = start >> 5;
  if (w < NW) {
    unsigned m = mask[w] & (0xffffffffu << (start & 31));
    if (m) return (w << 5) + __ffs(m) - 1;
    for (int k = w + 1; k < NW; ++k)
      if (mask[k]) return (k << 5) + __ffs(mask[k]) - 1;
  }
  return limit;
}
template <int NW>
__device__ __forceinline__ bool test_bit(const unsigned (&mask)[NW], int pos) {
  return pos >= 0 && (pos >> 5) < NW && ((mask[pos >> 5] >> (pos & 31)) & 1u);
}

template <int NW>
__device__ void assign_donors_serial(const float* saliency, const unsigned* sel_words, const unsigned* avail_words,
                                     int channels, int count, int* sources, int* donors) {
  unsigned selected[NW], available[NW];
#pragma unroll
  for (int k = 0; k < NW; ++k) {
    selected[k] = sel_words[k];
    available[k] = avail_words[k];
  }
  int n = 0;
#pragma unroll
  for (int k = 0; k < NW; ++k) {
    unsigned m = selected[k];
    while (m && n < count) {
      sources[n++] = (k << 5) + __ffs(m) - 1;
      m &= m - 1;
    }
  }
  for (int i = 0; i < count; ++i) {
    int source = sources[i];
    int low = test_bit<NW>(available, source - 1) ? source - 1 : -1;
    int high = (source + 1 < channels && test_bit<NW>(available, source + 1)) ? source + 1 : -1;
    if (low < 0 && high < 0) {
      // Ends of the contiguous salient run that contains the source.
      int left = source, right = source;
      while (test_bit<NW>(selected, left - 1)) --left;
      while (right + 1 < channels && test_bit<NW>(selected, right + 1)) ++right;
      int below = highest_below<NW>(available, left);
      int above = lowest_above<NW>(available, right, channels);
      int d_below = below >= 0 ? left - below : 0x7fffffff;
      int d_above = above < channels ? above - right : 0x7fffffff;
      if (d_below <= d_above) low = below;
      if (d_above <= d_below && above < channels) high = above;
    }
    int donor;
    if (low >= 0 && high >= 0)
      donor = saliency[low] <= saliency[high] ? low : high;  // ties: the lower channel
    else
      donor = low >= 0 ? low : high;
    if (donor < 0) donor = 0;  // unreachable for count <= channels/2
    donors[i] = donor;
    available[donor >> 5] &= ~(1u << (donor & 31));
  }
}

__device__ void select_donors_cta(const float* saliency, const float* error, bool use_error, int channels, int count,
                                  unsigned* rank_key, unsigned* sel_mask, unsigned* avail_mask, int* sources,
                                  int* donors) {
  const int c = threadIdx.x;
  const int words = (channels + 31) >> 5;
  if (c < kMaxWords) {
    sel_mask[c] = 0u;
    avail_mask[c] = 0u;
  }
  __syncthreads();
  bool selected = false;
  if (c < channels && count > 0) {
    // Non-negative floats order like their bit patterns; ties go to the lower channel.
    unsigned mine = __float_as_uint(saliency[c]);
    int rank = 0;
    for (int o = 0; o < channels; ++o) {
      unsigned other = __float_as_uint(saliency[o]);
      rank += (other > mine) || (other == mine && o < c);
    }
    selected = rank < count;
    if (selected) atomicOr(&sel_mask[c >> 5], 1u << (c & 31));
    if (use_error) rank_key[c] = selected ? 0x7f800000u : __float_as_uint(error[c]);
    if (!use_error && !selected) atomicOr(&avail_mask[c >> 5], 1u << (c & 31));
  }
  __syncthreads();
  if (use_error && c < channels && count > 0 && !selected) {
    unsigned mine = rank_key[c];
    int rank = 0;
    for (int o = 0; o < channels; ++o) {
      unsigned other = rank_key[o];
      rank += (other < mine) || (other == mine && o < c);
    }
    if (rank < count) atomicOr(&avail_mask[c >> 5], 1u << (c & 31));
  }
  __syncthreads();
  if (c == 0 && count > 0) {
    if (words <= 4)
      assign_donors_serial<4>(saliency, sel_mask, avail_mask, channels, count, sources, donors);
    else
      assign_donors_serial<kMaxWords>(saliency, sel_mask, avail_mask, channels, count, sources, donors);
  }
  __syncthreads();
}

// ------------------------------------------------------------------------------------------
struct K4Params {
  InputRef in;
  int sample_stride, count, min_error;
  FieldRef payload, scales, salient, donors, padding, roles;
  int descriptor_i32, role_bytes;
  int vector_path;  // 1: rows are 16-byte aligned and channels % 8 == 0
  int* status;
};

struct K4Shared {
  float* saliency;
  float* error;
  float* sampled_mean;
  float* scale;      // divisor per slot (the source's scale for a donor slot)
  int* read_from;    // channel whose value fills this slot
  int* kind;         // 0 normal, 1 salient (high nibble), 2 donor slot (low nibble of its source)
  unsigned* rank_key;
  unsigned* sel_mask;
  unsigned* avail_mask;
  int* sources;
  int* donors;
  double* rcp;
};

__host__ __device__ inline size_t k4_shared_bytes(int channels, int count, int tokens, bool min_error) {
  size_t bytes = 0;
  bytes += (size_t)channels * 4 * 7;          // saliency, error, sampled_mean, scale, read_from, kind, rank_key
  bytes += (size_t)kMaxWords * 4 * 2;         // masks
  bytes += (size_t)(count > 0 ? count : 1) * 4 * 2;
  bytes = (bytes + 7) & ~(size_t)7;
  if (min_error && tokens <= kRcpTable) bytes += (size_t)tokens * 8;
  return bytes;
}

__device__ inline K4Shared carve_k4_shared(unsigned char* raw, int channels, int count, int tokens, bool min_error) {
  K4Shared s;
  float* f = (float*)raw;
  s.saliency = f; f += channels;
  s.error = f; f += channels;
  s.sampled_mean = f; f += channels;
  s.scale = f; f += channels;
  s.read_from = (int*)f; f += channels;
  s.kind = (int*)f; f += channels;
  s.rank_key = (unsigned*)f; f += channels;
  s.sel_mask = (unsigned*)f; f += kMaxWords;
  s.avail_mask = (unsigned*)f; f += kMaxWords;
  s.sources = (int*)f; f += (count > 0 ? count : 1);
  s.donors = (int*)f; f += (count > 0 ? count : 1);
  size_t used = ((size_t)((unsigned char*)f - raw) + 7) & ~(size_t)7;
  s.rcp = (min_error && tokens <= kRcpTable) ? (double*)(raw + used) : nullptr;
  return s;
}

__device__ __forceinline__ unsigned encode_slot(float x, float scale, int kind) {
  float q = rintf(x / scale);
  if (kind == 0) return (unsigned)(int)(fminf(fmaxf(q, -7.f), 7.f) + 8.f);
  unsigned code = (unsigned)(int)(fminf(fmaxf(q, -127.f), 127.f) + 128.f);
  return kind == 1 ? (code >> 4) : (code & 15u);
}

template <typename T, int kMaxThreads>
__global__ void __launch_bounds__(kMaxThreads) k4_encode_kernel(K4Params p) {
  extern __shared__ __align__(16) unsigned char raw[];
  const int C = p.in.channels, tokens = p.in.tokens, count = p.count;
  K4Shared s = carve_k4_shared(raw, C, count, tokens, p.min_error != 0);
  const long long outer = blockIdx.x / p.in.n_inner, inner = blockIdx.x % p.in.n_inner;
  const long long slot = p.in.slot(outer);
  if (!p.in.slot_ok(slot)) {   // uniform over the CTA: nothing of this row is written
    if (threadIdx.x == 0) atomicOr(p.status, INQ_STATUS_BAD_INDEX);
    return;
  }
  const T* row = (const T*)p.in.x + outer * p.in.s_outer + inner * p.in.s_inner;
  const int c = threadIdx.x;

  if (s.rcp)
    for (int t = c; t < tokens; t += blockDim.x) s.rcp[t] = 1.0 / (double)(t + 1);
  __syncthreads();

  float absmax = 0.f;
  if (c < C) {
    ChannelStats st = channel_statistics<T>(row + c, p.in.s_token, tokens, p.sample_stride, p.min_error != 0, s.rcp);
    s.saliency[c] = st.saliency;
    s.sampled_mean[c] = st.sampled_mean;
    s.error[c] = st.donor_error;
    absmax = st.absmax;
    if (!st.finite) atomicOr(p.status, INQ_STATUS_NONFINITE);
    s.kind[c] = 0;
    s.read_from[c] = c;
  }
  __syncthreads();
  select_donors_cta(s.saliency, s.error, p.min_error != 0, C, count, s.rank_key, s.sel_mask, s.avail_mask,
                    s.sources, s.donors);

  if (c < C) {
    bool selected = (s.sel_mask[c >> 5] >> (c & 31)) & 1u;
    float own = fmaxf(absmax / (selected ? 127.0f : 7.0f), 1.17549435e-38f);
    s.scale[c] = own;
    ((float*)p.scales.at(slot, inner))[c] = own;
    if (selected) s.kind[c] = 1;
  }
  __syncthreads();
  if (c < count) {
    int source = s.sources[c], donor = s.donors[c];
    s.kind[donor] = 2;
    s.read_from[donor] = source;
    ((float*)p.padding.at(slot, inner))[c] = s.sampled_mean[donor];
    if (p.salient.base) {
      if (p.descriptor_i32) {
        ((int*)p.salient.at(slot, inner))[c] = source;
        ((int*)p.donors.at(slot, inner))[c] = donor;
      } else {
        ((unsigned char*)p.salient.at(slot, inner))[c] = (unsigned char)source;
        ((unsigned char*)p.donors.at(slot, inner))[c] = (unsigned char)donor;
      }
    }
  }
  __syncthreads();
  if (c < count) s.scale[s.donors[c]] = s.scale[s.sources[c]];  // a donor slot divides by its source's scale
  if (p.roles.base) {
    // role: donor channel of a salient channel, -1 for a normal one, -2-i for the i-th donor
    if (c < C) {
      int role = -1;
      for (int i = 0; i < count; ++i) {
        if (s.sources[i] == c) role = s.donors[i];
        if (s.donors[i] == c) role = -2 - i;
      }
      if (p.role_bytes == 1)
        ((signed char*)p.roles.at(slot, inner))[c] = (signed char)role;
      else
        ((short*)p.roles.at(slot, inner))[c] = (short)role;
    }
  }
  __syncthreads();

  unsigned char* payload = (unsigned char*)p.payload.at(slot, inner);
  const int row_bytes = C / 2;
  if (p.vector_path) {
    // A thread owns 8 fixed channels (4 payload bytes) and strides over tokens.
    const int chunks = C / 8;
    const int lanes = (blockDim.x / chunks) * chunks;
    if (c < lanes) {
      const int chunk = c % chunks, t0 = c / chunks, t_step = lanes / chunks;
      float scale[8];
      int kind[8], from[8];
      bool any_remote = false;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        int ch = chunk * 8 + j;
        scale[j] = s.scale[ch];
        kind[j] = s.kind[ch];
        from[j] = s.read_from[ch];
        any_remote |= (from[j] != ch);
      }
      for (int t = t0; t < tokens; t += t_step) {
        const T* src = row + (long long)t * p.in.s_token;
        float v[8];
        if (sizeof(T) == 2) {
          uint4 bits = *(const uint4*)(src + chunk * 8);
          const T* h = (const T*)&bits;
#pragma unroll
          for (int j = 0; j < 8; ++j) v[j] = to_float<T>(h[j]);
        } else {
          float4 a = *(const float4*)(src + chunk * 8), b = *(const float4*)(src + chunk * 8 + 4);
          v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
        }
        if (any_remote) {
#pragma unroll
          for (int j = 0; j < 8; ++j)
            if (kind[j] == 2) v[j] = to_float<T>(src[from[j]]);
        }
        unsigned word = 0;
#pragma unroll
        for (int j = 0; j < 8; ++j) word |= encode_slot(v[j], scale[j], kind[j]) << (4 * j);
        *(unsigned*)(payload + (long long)t * row_bytes + chunk * 4) = word;
      }
    }
  } else {
    for (long long idx = c; idx < (long long)tokens * row_bytes; idx += blockDim.x) {
      int t = (int)(idx / row_bytes), b = (int)(idx % row_bytes);
      const T* src = row + (long long)t * p.in.s_token;
      unsigned lo = encode_slot(to_float<T>(src[s.read_from[2 * b]]), s.scale[2 * b], s.kind[2 * b]);
      unsigned hi = encode_slot(to_float<T>(src[s.read_from[2 * b + 1]]), s.scale[2 * b + 1], s.kind[2 * b + 1]);
      payload[idx] = (unsigned char)(lo | (hi << 4));
    }
  }
}

// ------------------------------------------------------------------------------------------
// 128-channel fast path (every decode-capable layout): same arithmetic as k4_encode_kernel,
// fewer instructions per element.
//   * |x| maximum and the finite check come from one unsigned maximum of the fp32 bit patterns
//     (NaN and Inf sort above every finite value);
//   * x / s uses a correctly rounded reciprocal and two fused corrections, which returns the
//     IEEE quotient (Markstein); scales below 2^-100 keep the plain division;
//   * the selected / available sets are two 64-bit masks in registers.
struct Mask128 {
  unsigned long long lo, hi;
  __device__ __forceinline__ bool test(int i) const { return i >= 0 && i < 128 && (((i < 64 ? lo : hi) >> (i & 63)) & 1ull); }
  __device__ __forceinline__ void clear(int i) {
    if (i < 64) lo &= ~(1ull << i); else hi &= ~(1ull << (i - 64));
  }
  __device__ __forceinline__ int below(int pos) const {   // largest member < pos, or -1
    if (pos > 64) {
      unsigned long long m = pos >= 128 ? hi : (hi & ((1ull << (pos - 64)) - 1ull));
      if (m) return 127 - __clzll((long long)m);
      pos = 64;
    }
    unsigned long long m = pos >= 64 ? lo : (lo & ((1ull << pos) - 1ull));
    return m ? 63 - __clzll((long long)m) : -1;
  }
  __device__ __forceinline__ int above(int pos) const {   // smallest member > pos, or 128
    int start = pos + 1;
    if (start < 64) {
      unsigned long long m = lo & (~0ull << start);
      if (m) return __ffsll((long long)m) - 1;
      start = 64;
    }
    if (start >= 128) return 128;
    unsigned long long m = hi & (~0ull << (start - 64));
    return m ? 63 + __ffsll((long long)m) : 128;
  }
};

__device__ __forceinline__ float exact_quotient(float x, float s, float r, bool plain) {
  if (plain) return x / s;
  const float q0 = x * r;
  const float rem = fmaf(-q0, s, x);
  return fmaf(rem, r, q0);
}

__device__ __forceinline__ unsigned encode_slot_fast(float x, float scale, float rcp, bool plain, int kind) {
  const float q = rintf(exact_quotient(x, scale, rcp, plain));
  if (kind == 0) return (unsigned)(int)(fminf(fmaxf(q, -7.f), 7.f) + 8.f);
  const unsigned code = (unsigned)(int)(fminf(fmaxf(q, -127.f), 127.f) + 128.f);
  return kind == 1 ? (code >> 4) : (code & 15u);
}

template <typename T>
__device__ __forceinline__ unsigned f32_bits_of(T v) { return __float_as_uint(to_float<T>(v)); }

__device__ __forceinline__ void stage_copy16(void* dst, const void* src) {
  const unsigned d = (unsigned)__cvta_generic_to_shared(dst);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(src) : "memory");
}
__device__ __forceinline__ void stage_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void stage_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// REGULAR: tokens % 8 == 0 and sample_stride == 8.
// STAGED (16-bit inputs, contiguous rows, tokens % 32 == 0): the row's tokens stream twice -- once
// for the statistics, once for the packing -- through a ring of four 8 KB shared-memory stages
// filled by 16-byte asynchronous copies, three groups of 32 tokens in flight per CTA; every warp
// stages exactly the bytes it reads, so the two passes run without CTA-wide barriers.  A thread
// that fetches its own channel with 2-byte loads keeps only 16 bytes in flight, which left the
// kernel waiting on memory latency at a tenth of the HBM rate.
template <typename T, bool REGULAR, bool STAGED = false>
__global__ void __launch_bounds__(128, STAGED ? 5 : 7) k4_encode128_kernel(K4Params p) {
  constexpr int C = 128;
  constexpr int kGroupTokens = 32, kRing = 4;
  constexpr int kRowBytes = C * (int)sizeof(T);
  constexpr int kGroupBytes = kGroupTokens * kRowBytes;
  constexpr int kWarpStage = kGroupBytes / 4;   // a warp's share of a stage
  __shared__ __align__(16) unsigned char s_ring[STAGED ? kRing * kGroupBytes : 16];
  __shared__ float s_sal[C], s_err[C], s_mean[C], s_scale[C], s_rcp[C];
  __shared__ unsigned s_key[C];
  __shared__ unsigned char s_kind[C], s_from[C], s_plain[C];
  __shared__ int s_src[64], s_don[64];
  __shared__ unsigned s_sel[4], s_avail[4];
  __shared__ double s_inv[kRcpTable];
  const int tokens = p.in.tokens, count = p.count;
  const bool want_error = p.min_error != 0;
  const long long outer = blockIdx.x / p.in.n_inner, inner = blockIdx.x % p.in.n_inner;
  const long long slot = p.in.slot(outer);
  if (!p.in.slot_ok(slot)) {   // uniform over the CTA: nothing of this row is written
    if (threadIdx.x == 0) atomicOr(p.status, INQ_STATUS_BAD_INDEX);
    return;
  }
  const T* row = (const T*)p.in.x + outer * p.in.s_outer + inner * p.in.s_inner;
  const int c = threadIdx.x;
  if (want_error)
    for (int t = c; t < tokens; t += C) s_inv[t] = 1.0 / (double)(t + 1);
  if (c < 4) s_sel[c] = s_avail[c] = 0u;
  __syncthreads();

  // ---- statistics: one thread per channel, sequential over tokens
  unsigned top_bits = 0u;
  CascadePair cascade;
  const int samples = (tokens + p.sample_stride - 1) / p.sample_stride;
  cascade.init(samples);
  double mean = 0.0, m2 = 0.0, count_d = 0.0;
  int next_sample = 0;
  {
    const T* column = row + c;
    constexpr int kUnroll = 8;
    const long long step = p.in.s_token;
    // the next batch of tokens is requested before the current one is consumed, so the
    // sequential (Welford) chain never waits on a freshly issued load
    T ahead[kUnroll];
    if constexpr (STAGED) {
      // Every warp stages what it reads itself, so the passes need no CTA-wide barrier: for the
      // statistics the 64 bytes of its 32 channels in each of the group's 32 token rows.
      const int n_groups = tokens / kGroupTokens;
      const int warp_id = c >> 5, lane_id = c & 31;
      unsigned char* const warp_ring = s_ring + warp_id * (kRing * kWarpStage);
      const unsigned char* src_bytes = (const unsigned char*)row;
      auto issue = [&](int step_index) {
        if (step_index < 2 * n_groups) {
          unsigned char* dst = warp_ring + (step_index & (kRing - 1)) * kWarpStage;
          if (step_index < n_groups) {
            const unsigned char* src = src_bytes + (long long)step_index * kGroupBytes + warp_id * 64;
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              const int idx = k * 32 + lane_id, token = idx >> 2, part = idx & 3;
              stage_copy16(dst + token * 64 + part * 16, src + token * kRowBytes + part * 16);
            }
          } else {
            // packing: the thread's own 16 bytes of token rows 2 * warp + lane / 16 + 8k
            const unsigned char* src = src_bytes + (long long)(step_index - n_groups) * kGroupBytes;
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              const int token = 2 * warp_id + (lane_id >> 4) + 8 * k;
              stage_copy16(dst + (2 * k + (lane_id >> 4)) * kRowBytes + (lane_id & 15) * 16,
                           src + token * kRowBytes + (lane_id & 15) * 16);
            }
          }
        }
        stage_commit();
      };
      issue(0);
      issue(1);
      issue(2);
      const double* inv = s_inv;
      for (int g = 0; g < n_groups; ++g) {
        stage_wait<kRing - 2>();
        __syncwarp();   // group g has landed for every lane; the stage of group g - 1 is free
        issue(g + 3);
        const T* tile = (const T*)(warp_ring + (g & (kRing - 1)) * kWarpStage) + lane_id;
#pragma unroll
        for (int b = 0; b < kGroupTokens / kUnroll; ++b) {
          float v[kUnroll];
#pragma unroll
          for (int u = 0; u < kUnroll; ++u) v[u] = to_float<T>(tile[(b * kUnroll + u) * 32]);
          cascade.add(v[0]);   // every eighth token is a sample
#pragma unroll
          for (int u = 0; u < kUnroll; ++u) {
            const float x = v[u];
            top_bits = max(top_bits, __float_as_uint(x) & 0x7fffffffu);
            if (want_error) {
              const double xd = (double)x;
              const double delta = xd - mean;
              count_d = count_d + 1.0;
              mean = mean + divide_by_count(delta, count_d, inv[u]);
              m2 = m2 + delta * (xd - mean);
            }
          }
          inv += kUnroll;
        }
      }
      (void)step;
      (void)ahead;
    } else if (REGULAR) {
      const T* cursor = column;
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) ahead[u] = cursor[u * step];
      const double* inv = s_inv;
      for (int base = 0; base < tokens; base += kUnroll) {
        float v[kUnroll];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) v[u] = to_float<T>(ahead[u]);
        cursor += kUnroll * step;
        if (base + kUnroll < tokens) {
#pragma unroll
          for (int u = 0; u < kUnroll; ++u) ahead[u] = cursor[u * step];
        }
        cascade.add(v[0]);   // every eighth token is a sample
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
          const float x = v[u];
          top_bits = max(top_bits, __float_as_uint(x) & 0x7fffffffu);
          if (want_error) {
            const double xd = (double)x;
            const double delta = xd - mean;
            count_d = count_d + 1.0;
            mean = mean + divide_by_count(delta, count_d, inv[u]);
            m2 = m2 + delta * (xd - mean);
          }
        }
        inv += kUnroll;
      }
    } else {
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) ahead[u] = u < tokens ? column[(long long)u * p.in.s_token] : T();
    for (int base = 0; base < tokens; base += kUnroll) {
      float v[kUnroll];
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) v[u] = to_float<T>(ahead[u]);
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        const int t = base + kUnroll + u;
        if (t < tokens) ahead[u] = column[(long long)t * p.in.s_token];
      }
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        const int t = base + u;
        if (t < tokens) {
          const float x = v[u];
          top_bits = max(top_bits, __float_as_uint(x) & 0x7fffffffu);
          if (t == next_sample) {
            cascade.add(x);
            next_sample += p.sample_stride;
          }
          if (want_error) {
            const double xd = (double)x;
            const double delta = xd - mean;
            count_d = count_d + 1.0;
            mean = mean + divide_by_count(delta, count_d, s_inv[t]);
            m2 = m2 + delta * (xd - mean);
          }
        }
      }
    }
    }
  }
  float abs_total, sum_total;
  cascade.finish(abs_total, sum_total);
  const float saliency = abs_total / (float)samples, sampled_mean = sum_total / (float)samples;
  float donor_error = 0.f;
  if (want_error) {
    const float variance = (float)(m2 / (double)tokens);
    const float diff = (float)mean - sampled_mean;
    donor_error = variance + diff * diff;
  }
  if (top_bits >= 0x7f800000u) atomicOr(p.status, INQ_STATUS_NONFINITE);
  const float absmax = __uint_as_float(top_bits);
  s_sal[c] = saliency;
  s_mean[c] = sampled_mean;
  s_err[c] = donor_error;
  __syncthreads();

  // ---- top-`count` channels by saliency (ties: lower channel), optional least-error pool
  bool selected = false;
  if (count > 0) {
    const unsigned mine = __float_as_uint(saliency);
    int rank = 0;
#pragma unroll 4
    for (int o4 = 0; o4 < C / 4; ++o4) {
      const float4 f = *(const float4*)(s_sal + 4 * o4);
      const unsigned k0 = __float_as_uint(f.x), k1 = __float_as_uint(f.y), k2 = __float_as_uint(f.z), k3 = __float_as_uint(f.w);
      rank += (k0 > mine) || (k0 == mine && 4 * o4 + 0 < c);
      rank += (k1 > mine) || (k1 == mine && 4 * o4 + 1 < c);
      rank += (k2 > mine) || (k2 == mine && 4 * o4 + 2 < c);
      rank += (k3 > mine) || (k3 == mine && 4 * o4 + 3 < c);
    }
    selected = rank < count;
    if (selected) atomicOr(&s_sel[c >> 5], 1u << (c & 31));
    s_key[c] = selected ? 0x7f800000u : __float_as_uint(donor_error);
    if (!want_error && !selected) atomicOr(&s_avail[c >> 5], 1u << (c & 31));
  }
  __syncthreads();
  if (want_error && count > 0 && !selected) {
    const unsigned mine = s_key[c];
    int rank = 0;
#pragma unroll 4
    for (int o4 = 0; o4 < C / 4; ++o4) {
      const uint4 k = *(const uint4*)(s_key + 4 * o4);
      rank += (k.x < mine) || (k.x == mine && 4 * o4 + 0 < c);
      rank += (k.y < mine) || (k.y == mine && 4 * o4 + 1 < c);
      rank += (k.z < mine) || (k.z == mine && 4 * o4 + 2 < c);
      rank += (k.w < mine) || (k.w == mine && 4 * o4 + 3 < c);
    }
    if (rank < count) atomicOr(&s_avail[c >> 5], 1u << (c & 31));
  }
  __syncthreads();
  if (c == 0 && count > 0) {
    Mask128 sel{(unsigned long long)s_sel[0] | ((unsigned long long)s_sel[1] << 32),
                (unsigned long long)s_sel[2] | ((unsigned long long)s_sel[3] << 32)};
    Mask128 avail{(unsigned long long)s_avail[0] | ((unsigned long long)s_avail[1] << 32),
                  (unsigned long long)s_avail[2] | ((unsigned long long)s_avail[3] << 32)};
    int n = 0;
    for (unsigned long long m = sel.lo; m && n < count; m &= m - 1) s_src[n++] = __ffsll((long long)m) - 1;
    for (unsigned long long m = sel.hi; m && n < count; m &= m - 1) s_src[n++] = 63 + __ffsll((long long)m);
    for (int i = 0; i < count; ++i) {
      const int source = s_src[i];
      int low = avail.test(source - 1) ? source - 1 : -1;
      int high = avail.test(source + 1) ? source + 1 : -1;
      if (low < 0 && high < 0) {
        int left = source, right = source;
        while (sel.test(left - 1)) --left;
        while (sel.test(right + 1)) ++right;
        const int below = avail.below(left), above = avail.above(right);
        const int d_below = below >= 0 ? left - below : 0x7fffffff;
        const int d_above = above < 128 ? above - right : 0x7fffffff;
        if (d_below <= d_above) low = below;
        if (d_above <= d_below && above < 128) high = above;
      }
      int donor;
      if (low >= 0 && high >= 0)
        donor = s_sal[low] <= s_sal[high] ? low : high;
      else
        donor = low >= 0 ? low : high;
      if (donor < 0) donor = 0;
      s_don[i] = donor;
      avail.clear(donor);
    }
  }
  // ---- scales and per-slot encoding parameters
  const float own_scale = fmaxf(absmax / (selected ? 127.0f : 7.0f), 1.17549435e-38f);
  s_scale[c] = own_scale;
  s_rcp[c] = __frcp_rn(own_scale);
  s_plain[c] = own_scale < 7.8886091e-31f;   // 2^-100: remainders would underflow
  s_kind[c] = selected ? 1 : 0;
  s_from[c] = (unsigned char)c;
  ((float*)p.scales.at(slot, inner))[c] = own_scale;
  __syncthreads();
  if (c < count) {
    const int source = s_src[c], donor = s_don[c];
    s_kind[donor] = 2;
    s_from[donor] = (unsigned char)source;
    ((float*)p.padding.at(slot, inner))[c] = s_mean[donor];
    if (p.salient.base) {
      ((unsigned char*)p.salient.at(slot, inner))[c] = (unsigned char)source;
      ((unsigned char*)p.donors.at(slot, inner))[c] = (unsigned char)donor;
    }
  }
  __syncthreads();
  if (p.roles.base) {
    int role = -1;
    for (int i = 0; i < count; ++i) {
      if (s_src[i] == c) role = s_don[i];
      if (s_don[i] == c) role = -2 - i;
    }
    if (p.role_bytes == 1)
      ((signed char*)p.roles.at(slot, inner))[c] = (signed char)role;
    else
      ((short*)p.roles.at(slot, inner))[c] = (short)role;
  }
  // ---- packing: a thread owns 8 fixed slots (4 payload bytes) and strides over tokens
  unsigned char* payload = (unsigned char*)p.payload.at(slot, inner);
  const int chunk = c & 15, t0 = c >> 4;
  // per slot: divisor, clamp limit, bias and which nibble of the code is stored -- a normal slot
  // keeps clamp(q, +-7) + 8, a salient slot the high nibble of clamp(q, +-127) + 128, a donor slot
  // the low nibble of its source's code; all three are (code >> shift) & 15
  float scale[8], rcp[8], limit[8], bias[8];
  int shift[8], from[8], kind[8];
  bool any_plain = false, any_remote = false;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const int ch = chunk * 8 + j;
    kind[j] = s_kind[ch];
    from[j] = s_from[ch];
    const int src_ch = from[j];       // a donor slot divides its source's value by its source's scale
    scale[j] = s_scale[src_ch];
    rcp[j] = s_rcp[src_ch];
    any_plain |= s_plain[src_ch] != 0;
    limit[j] = kind[j] ? 127.f : 7.f;
    bias[j] = kind[j] ? 128.f : 8.f;
    shift[j] = kind[j] == 1 ? 4 : 0;
    any_remote |= (from[j] != ch);
  }
  if constexpr (STAGED) {
    const int n_groups = tokens / kGroupTokens;
    const int warp_id = c >> 5, lane_id = c & 31;
    unsigned char* const warp_ring = s_ring + warp_id * (kRing * kWarpStage);
    const unsigned char* src_bytes = (const unsigned char*)row;
    for (int g = 0; g < n_groups; ++g) {
      const int step_index = n_groups + g;
      stage_wait<kRing - 2>();
      __syncwarp();
      if (step_index + 3 < 2 * n_groups) {
        unsigned char* dst = warp_ring + ((step_index + 3) & (kRing - 1)) * kWarpStage;
        const unsigned char* src = src_bytes + (long long)(g + 3) * kGroupBytes;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const int token = 2 * warp_id + (lane_id >> 4) + 8 * k;
          stage_copy16(dst + (2 * k + (lane_id >> 4)) * kRowBytes + (lane_id & 15) * 16,
                       src + token * kRowBytes + (lane_id & 15) * 16);
        }
      }
      stage_commit();
      const unsigned char* tile = warp_ring + (step_index & (kRing - 1)) * kWarpStage;
#pragma unroll
      for (int i = 0; i < kGroupTokens / 8; ++i) {
        const int tl = t0 + 8 * i;   // t0 = 2 * warp + lane / 16
        const T* trow = (const T*)(tile + (2 * i + (lane_id >> 4)) * kRowBytes);
        const uint4 cur = *(const uint4*)(trow + chunk * 8);
        const T* hv = (const T*)&cur;
        float v[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = to_float<T>(hv[j]);
        if (any_remote) {
#pragma unroll
          for (int j = 0; j < 8; ++j)
            if (kind[j] == 2) v[j] = to_float<T>(trow[from[j]]);
        }
        unsigned word = 0;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float q = rintf(exact_quotient(v[j], scale[j], rcp[j], any_plain));
          const unsigned code = (unsigned)(int)(fminf(fmaxf(q, -limit[j]), limit[j]) + bias[j]);
          word |= ((code >> shift[j]) & 15u) << (4 * j);
        }
        *(unsigned*)(payload + (long long)(g * kGroupTokens + tl) * 64 + chunk * 4) = word;
      }
    }
    stage_wait<0>();
    return;
  }
  constexpr int kVec = sizeof(T) == 2 ? 1 : 2;   // 16-byte vectors per 8 elements
  uint4 next[kVec];
  if (t0 < tokens) {
#pragma unroll
    for (int q = 0; q < kVec; ++q) next[q] = ((const uint4*)(row + (long long)t0 * p.in.s_token + chunk * 8))[q];
  }
  const long long pack_step = 8 * p.in.s_token;
  const T* src = row + (long long)t0 * p.in.s_token - pack_step;
  unsigned char* dst = payload + (long long)t0 * 64 + chunk * 4 - 512;
  for (int t = t0; t < tokens; t += 8) {
    src += pack_step;
    dst += 512;
    uint4 cur[kVec];
#pragma unroll
    for (int q = 0; q < kVec; ++q) cur[q] = next[q];
    if (t + 8 < tokens) {
#pragma unroll
      for (int q = 0; q < kVec; ++q) next[q] = ((const uint4*)(src + pack_step + chunk * 8))[q];
    }
    float v[8];
    const T* hv = (const T*)cur;
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = to_float<T>(hv[j]);
    if (any_remote) {
#pragma unroll
      for (int j = 0; j < 8; ++j)
        if (kind[j] == 2) v[j] = to_float<T>(src[from[j]]);
    }
    unsigned word = 0;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float q = rintf(exact_quotient(v[j], scale[j], rcp[j], any_plain));
      const unsigned code = (unsigned)(int)(fminf(fmaxf(q, -limit[j]), limit[j]) + bias[j]);
      word |= ((code >> shift[j]) & 15u) << (4 * j);
    }
    *(unsigned*)dst = word;
  }
}

template <typename T>
__global__ void __launch_bounds__(1024) k4_statistics_kernel(InputRef in, int sample_stride, float* saliency,
                                                              float* sampled_mean, float* donor_error, float* absmax) {
  extern __shared__ __align__(16) unsigned char raw[];
  double* rcp = (donor_error && in.tokens <= kRcpTable) ? (double*)raw : nullptr;
  const long long outer = blockIdx.x / in.n_inner, inner = blockIdx.x % in.n_inner;
  const T* row = (const T*)in.x + outer * in.s_outer + inner * in.s_inner;
  if (rcp)
    for (int t = threadIdx.x; t < in.tokens; t += blockDim.x) rcp[t] = 1.0 / (double)(t + 1);
  __syncthreads();
  const int c = threadIdx.x;
  if (c >= in.channels) return;
  ChannelStats st = channel_statistics<T>(row + c, in.s_token, in.tokens, sample_stride, donor_error != nullptr, rcp);
  long long o = (long long)blockIdx.x * in.channels + c;
  if (saliency) saliency[o] = st.saliency;
  if (sampled_mean) sampled_mean[o] = st.sampled_mean;
  if (donor_error) donor_error[o] = st.donor_error;
  if (absmax) absmax[o] = st.absmax;
}

__global__ void __launch_bounds__(1024) select_kernel(const float* saliency, const float* error, int channels, int count,
                                                       long long* sources, long long* donors) {
  extern __shared__ __align__(16) unsigned char raw[];
  float* sal = (float*)raw;
  float* err = sal + channels;
  unsigned* rank_key = (unsigned*)(err + channels);
  unsigned* sel_mask = rank_key + channels;
  unsigned* avail_mask = sel_mask + kMaxWords;
  int* src = (int*)(avail_mask + kMaxWords);
  int* don = src + count;
  const long long row = blockIdx.x;
  const int c = threadIdx.x;
  if (c < channels) {
    sal[c] = saliency[row * channels + c];
    err[c] = error ? error[row * channels + c] : 0.f;
  }
  __syncthreads();
  select_donors_cta(sal, err, error != nullptr, channels, count, rank_key, sel_mask, avail_mask, src, don);
  if (c < count) {
    sources[row * count + c] = src[c];
    donors[row * count + c] = don[c];
  }
}

// ------------------------------------------------------------------------------------------
// 128-channel rows, 16-bit output: a thread owns 8 consecutive channels of one token (4 payload bytes
// in, 16 bytes out); 16 threads cover a token, a CTA of 256 threads covers 16 tokens per step.
template <typename T>
__global__ void __launch_bounds__(256) k4_dequantize128_kernel(const unsigned char* payload, const float* scales, const void* salient,
                                                               const void* donors, const float* padding, int tokens, int count, T* out,
                                                               int rows_inner, long long out_so, long long out_si) {
  __shared__ int role[128];
  __shared__ float scale[128], pad[128];
  const long long row = blockIdx.x;
  if (threadIdx.x < 128) {
    role[threadIdx.x] = -1;
    scale[threadIdx.x] = scales[row * 128 + threadIdx.x];
    pad[threadIdx.x] = 0.f;
  }
  __syncthreads();
  if ((int)threadIdx.x < count) {
    const int i = threadIdx.x;
    const int s = ((const unsigned char*)salient)[row * count + i], d = ((const unsigned char*)donors)[row * count + i];
    role[s] = d;
    role[d] = -2 - i;
    pad[d] = padding[row * count + i];
  }
  __syncthreads();
  const unsigned char* bytes = payload + row * (long long)tokens * 64;
  T* dst = out + (row / rows_inner) * out_so + (row % rows_inner) * out_si;
  const int c0 = (threadIdx.x & 15) * 8;
  int r[8];
  float sc[8], pd[8];
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    r[k] = role[c0 + k];
    sc[k] = scale[c0 + k];
    pd[k] = pad[c0 + k];
  }
  const int per_cta = (tokens + gridDim.y - 1) / gridDim.y;
  const int t_begin = blockIdx.y * per_cta, t_end = min(tokens, t_begin + per_cta);
  for (int t = t_begin + (threadIdx.x >> 4); t < t_end; t += 16) {
    const unsigned char* line = bytes + (long long)t * 64;
    const unsigned word = *(const unsigned*)(line + (c0 >> 1));
    T vals[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const int slot = (word >> (4 * k)) & 15;
      float value;
      if (r[k] >= 0) {
        const int partner = (line[r[k] >> 1] >> ((r[k] & 1) * 4)) & 15;
        value = (float)(((slot << 4) | partner) - 128) * sc[k];
      } else if (r[k] == -1) {
        value = (float)(slot - 8) * sc[k];
      } else {
        value = pd[k];
      }
      vals[k] = from_float<T>(value);
    }
    *(uint4*)(dst + (long long)t * 128 + c0) = *(const uint4*)vals;
  }
}

template <typename T>
__global__ void k4_dequantize_kernel(const unsigned char* payload, const float* scales, const void* salient,
                                     const void* donors, int descriptor_i32, const float* padding, int tokens,
                                     int channels, int count, T* out, int rows_inner, long long out_so, long long out_si) {
  extern __shared__ __align__(16) unsigned char raw[];
  int* role = (int*)raw;  // >=0 partner slot of a salient channel, -1 normal, <=-2 donor
  float* scale = (float*)(role + channels);
  float* pad = scale + channels;
  const long long row = blockIdx.x;
  for (int c = threadIdx.x; c < channels; c += blockDim.x) {
    role[c] = -1;
    scale[c] = scales[row * channels + c];
    pad[c] = 0.f;
  }
  __syncthreads();
  for (int i = threadIdx.x; i < count; i += blockDim.x) {
    int s = descriptor_i32 ? ((const int*)salient)[row * count + i] : ((const unsigned char*)salient)[row * count + i];
    int d = descriptor_i32 ? ((const int*)donors)[row * count + i] : ((const unsigned char*)donors)[row * count + i];
    role[s] = d;
    role[d] = -2 - i;
    pad[d] = padding[row * count + i];
  }
  __syncthreads();
  const unsigned char* bytes = payload + row * (long long)tokens * (channels / 2);
  // row (outer, inner) lands at out + outer * out_so + inner * out_si (elements); its tokens are contiguous
  T* dst = out + (row / rows_inner) * out_so + (row % rows_inner) * out_si;
  const int t_begin = blockIdx.y * 16, t_end = min(tokens, t_begin + 16);
  for (int idx = t_begin * channels + threadIdx.x; idx < t_end * channels; idx += blockDim.x) {
    int t = idx / channels, c = idx % channels;
    const unsigned char* line = bytes + (long long)t * (channels / 2);
    int slot = (line[c >> 1] >> ((c & 1) * 4)) & 15;
    int r = role[c];
    float value;
    if (r >= 0) {
      int partner = (line[r >> 1] >> ((r & 1) * 4)) & 15;
      value = (float)(((slot << 4) | partner) - 128) * scale[c];
    } else if (r == -1) {
      value = (float)(slot - 8) * scale[c];
    } else {
      value = pad[c];
    }
    dst[idx] = from_float<T>(value);
  }
}

// ------------------------------------------------------------------------------------------
struct VParams {
  InputRef in;
  int bits, group;
  FieldRef payload, scales, offsets;
  int* status;
};

// One warp per token row; a lane owns channels / 32 consecutive channels.
template <typename T, int CPL>
__global__ void __launch_bounds__(256) v_encode_kernel(VParams p) {
  const int warps_per_block = blockDim.x / 32, warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  const long long outer = blockIdx.x / p.in.n_inner, inner = blockIdx.x % p.in.n_inner;
  const long long slot = p.in.slot(outer);
  if (!p.in.slot_ok(slot)) {   // uniform over the CTA: nothing of this row is written
    if (threadIdx.x == 0) atomicOr(p.status, INQ_STATUS_BAD_INDEX);
    return;
  }
  const int t = blockIdx.y * warps_per_block + warp;
  if (t >= p.in.tokens) return;
  const int C = p.in.channels, groups = C / p.group;
  const T* src = (const T*)p.in.x + outer * p.in.s_outer + inner * p.in.s_inner + (long long)t * p.in.s_token + lane * CPL;
  float v[CPL];
#pragma unroll
  for (int j = 0; j < CPL; ++j) v[j] = to_float<T>(src[j]);
  float lo = v[0], hi = v[0];
  bool finite = true;
#pragma unroll
  for (int j = 0; j < CPL; ++j) {
    lo = fminf(lo, v[j]);
    hi = fmaxf(hi, v[j]);
    finite = finite && finite_f32(v[j]);
  }
  const int lanes_per_group = p.group / CPL;
  for (int off = 1; off < lanes_per_group; off <<= 1) {
    lo = fminf(lo, __shfl_xor_sync(0xffffffffu, lo, off));
    hi = fmaxf(hi, __shfl_xor_sync(0xffffffffu, hi, off));
  }
  const float levels = (float)((1 << p.bits) - 1);
  __half offset16 = __float2half_rn(lo);
  __half scale16 = __float2half_rn(fmaxf((hi - lo) / levels, 6.103515625e-05f));
  float offset = __half2float(offset16), scale = __half2float(scale16);
  finite = finite && finite_f32(offset) && finite_f32(scale);
  if (!finite) atomicOr(p.status, INQ_STATUS_NONFINITE);
  const int g = lane / lanes_per_group;
  if (lane % lanes_per_group == 0) {
    ((__half*)p.scales.at(slot, inner))[(long long)t * groups + g] = scale16;
    ((__half*)p.offsets.at(slot, inner))[(long long)t * groups + g] = offset16;
  }
  // Pack this lane's codes, then OR together the lanes that share a 32-bit word.
  const int bits = p.bits, lane_bits = CPL * bits;
  unsigned char* dst = (unsigned char*)p.payload.at(slot, inner) + (long long)t * (C * bits / 8);
  if (lane_bits >= 32) {
    constexpr int kWords = (CPL * 4 + 31) / 32;  // upper bound for bits = 4
    unsigned words[kWords];
#pragma unroll
    for (int w = 0; w < kWords; ++w) words[w] = 0u;
#pragma unroll
    for (int j = 0; j < CPL; ++j) {
      unsigned code = (unsigned)(int)fminf(fmaxf(rintf((v[j] - offset) / scale), 0.f), levels);
      words[(j * bits) >> 5] |= code << ((j * bits) & 31);
    }
    const int n_words = lane_bits / 32;
    for (int w = 0; w < n_words; ++w) ((unsigned*)dst)[lane * n_words + w] = words[w];
  } else {
    unsigned word = 0u;
    const int lanes_per_word = 32 / lane_bits;
#pragma unroll
    for (int j = 0; j < CPL; ++j) {
      unsigned code = (unsigned)(int)fminf(fmaxf(rintf((v[j] - offset) / scale), 0.f), levels);
      word |= code << (((lane % lanes_per_word) * CPL + j) * bits);
    }
    for (int off = 1; off < lanes_per_word; off <<= 1) word |= __shfl_xor_sync(0xffffffffu, word, off);
    if (lane % lanes_per_word == 0) ((unsigned*)dst)[lane / lanes_per_word] = word;
  }
}

// 128-channel fast path of the value encoder: a warp owns 8 consecutive tokens, issues all its
// loads first (2 KB in flight per warp), then quantises token by token.  A lane owns 4 channels.
template <typename T, int BITS, int GROUP>
__global__ void __launch_bounds__(256) v_encode128_kernel(VParams p) {
  constexpr int kRows = 8;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long outer = blockIdx.x / p.in.n_inner, inner = blockIdx.x % p.in.n_inner;
  const long long slot = p.in.slot(outer);
  if (!p.in.slot_ok(slot)) {   // uniform over the CTA: nothing of this row is written
    if (threadIdx.x == 0) atomicOr(p.status, INQ_STATUS_BAD_INDEX);
    return;
  }
  const int t0 = (blockIdx.y * 8 + warp) * kRows;
  if (t0 >= p.in.tokens) return;
  const T* base = (const T*)p.in.x + outer * p.in.s_outer + inner * p.in.s_inner + lane * 4;
  float v[kRows][4];
#pragma unroll
  for (int k = 0; k < kRows; ++k) {
    const int t = min(t0 + k, p.in.tokens - 1);
    const T* src = base + (long long)t * p.in.s_token;
    if (sizeof(T) == 2) {
      const uint2 bits = *(const uint2*)src;
      const T* hv = (const T*)&bits;
#pragma unroll
      for (int j = 0; j < 4; ++j) v[k][j] = to_float<T>(hv[j]);
    } else {
      const float4 f = *(const float4*)src;
      v[k][0] = f.x; v[k][1] = f.y; v[k][2] = f.z; v[k][3] = f.w;
    }
  }
  constexpr int lanes_per_group = GROUP / 4, groups = 128 / GROUP, bits = BITS;
  constexpr float levels = (float)((1 << BITS) - 1);
  unsigned nonfinite = 0u;
  unsigned char* payload = (unsigned char*)p.payload.at(slot, inner);
  __half* scales = (__half*)p.scales.at(slot, inner);
  __half* offsets = (__half*)p.offsets.at(slot, inner);
#pragma unroll
  for (int k = 0; k < kRows; ++k) {
    const int t = t0 + k;
    if (t >= p.in.tokens) break;
    float lo = fminf(fminf(v[k][0], v[k][1]), fminf(v[k][2], v[k][3]));
    float hi = fmaxf(fmaxf(v[k][0], v[k][1]), fmaxf(v[k][2], v[k][3]));
    unsigned top = max(max(__float_as_uint(v[k][0]) & 0x7fffffffu, __float_as_uint(v[k][1]) & 0x7fffffffu),
                       max(__float_as_uint(v[k][2]) & 0x7fffffffu, __float_as_uint(v[k][3]) & 0x7fffffffu));
#pragma unroll
    for (int off = 1; off < lanes_per_group; off <<= 1) {
      lo = fminf(lo, __shfl_xor_sync(0xffffffffu, lo, off));
      hi = fmaxf(hi, __shfl_xor_sync(0xffffffffu, hi, off));
    }
    const __half offset16 = __float2half_rn(lo);
    const __half scale16 = __float2half_rn(fmaxf((hi - lo) / levels, 6.103515625e-05f));
    const float offset = __half2float(offset16), scale = __half2float(scale16);
    top = max(top, max(__float_as_uint(offset) & 0x7fffffffu, __float_as_uint(scale) & 0x7fffffffu));
    nonfinite |= top >= 0x7f800000u;
    if (lane % lanes_per_group == 0) {
      const int g = lane / lanes_per_group;
      scales[(long long)t * groups + g] = scale16;
      offsets[(long long)t * groups + g] = offset16;
    }
    // stored scales are >= 2^-14, so the fused-correction quotient is the IEEE quotient
    const float rcp = __frcp_rn(scale);
    unsigned word = 0u;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float q = exact_quotient(v[k][j] - offset, scale, rcp, false);
      const unsigned code = (unsigned)(int)fminf(fmaxf(rintf(q), 0.f), levels);
      word |= code << (j * bits);
    }
    if (bits == 2) {
      // 8 bits per lane, four lanes per 32-bit word
      word <<= 8 * (lane & 3);
      word |= __shfl_xor_sync(0xffffffffu, word, 1);
      word |= __shfl_xor_sync(0xffffffffu, word, 2);
      if ((lane & 3) == 0) ((unsigned*)(payload + (long long)t * 32))[lane >> 2] = word;
    } else {
      word <<= 16 * (lane & 1);
      word |= __shfl_xor_sync(0xffffffffu, word, 1);
      if ((lane & 1) == 0) ((unsigned*)(payload + (long long)t * 64))[lane >> 1] = word;
    }
  }
  if (nonfinite) atomicOr(p.status, INQ_STATUS_NONFINITE);
}

template <typename T>
__global__ void v_dequantize_kernel(const unsigned char* payload, const __half* scales, const __half* offsets,
                                    long long total, int channels, int bits, int group, T* out, int tokens, int rows_inner,
                                    long long out_so, long long out_si) {
  long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  long long token = idx / channels;
  int c = (int)(idx % channels);
  int per_byte = 8 / bits;
  unsigned byte = payload[token * (channels / per_byte) + c / per_byte];
  float code = (float)((byte >> ((c % per_byte) * bits)) & ((1u << bits) - 1u));
  long long param = token * (channels / group) + c / group;
  float value = code * __half2float(scales[param]);
  value = value + __half2float(offsets[param]);
  // row (outer, inner) lands at out + outer * out_so + inner * out_si (elements); its tokens are contiguous
  const long long row = token / tokens;
  out[(row / rows_inner) * out_so + (row % rows_inner) * out_si + (token % tokens) * channels + c] = from_float<T>(value);
}

// 128 channels, 16-bit output: a thread owns 8 consecutive channels of one token (they share a group)
template <typename T, int BITS>
__global__ void __launch_bounds__(256) v_dequantize128_kernel(const unsigned char* payload, const __half* scales, const __half* offsets,
                                                              long long total_tokens, int tokens, int group, T* out, int rows_inner,
                                                              long long out_so, long long out_si) {
  const long long item = (long long)blockIdx.x * blockDim.x + threadIdx.x;   // (token, chunk of 8 channels)
  const long long token = item >> 4;
  if (token >= total_tokens) return;
  const int c0 = (int)(item & 15) * 8;
  constexpr int kBytes = BITS;   // 8 channels x BITS bits
  const unsigned char* src = payload + token * (128 * BITS / 8) + (c0 * BITS / 8);
  unsigned word = 0;
#pragma unroll
  for (int b = 0; b < kBytes; ++b) word |= (unsigned)src[b] << (8 * b);
  const int groups = 128 / group;
  const long long param = token * groups + c0 / group;
  const float sc = __half2float(scales[param]), of = __half2float(offsets[param]);
  T vals[8];
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    const float code = (float)((word >> (BITS * k)) & ((1u << BITS) - 1u));
    float value = code * sc;
    value = value + of;
    vals[k] = from_float<T>(value);
  }
  const long long row = token / tokens;
  T* dst = out + (row / rows_inner) * out_so + (row % rows_inner) * out_si + (token % tokens) * 128 + c0;
  *(uint4*)dst = *(const uint4*)vals;
}

// All sealed blocks of one cached layer back into a dense history in ONE launch, addressed through the
// decode descriptors of that layer: the 6-pointer table (key payload, key scales, key padding, value
// payload, value scales, value offsets per block) and the int8 role map.  CTA (block-head row, token
// part): keys exactly as k4_dequantize128_kernel, 2-bit values in groups of 64 channels exactly as
// v_dequantize128_kernel; a thread owns 8 consecutive channels of a token.  Rows land at
// out + head * stride_h + (position + block * tokens + t) * 128.
template <typename T>
__global__ void __launch_bounds__(256) restore_table_kernel(const long long* table, const signed char* roles, int heads, int tokens,
                                                            int count, T* out_k, T* out_v, long long stride_h, long long position) {
  __shared__ int role[128];
  __shared__ float scale[128], pad[128];
  const int b = blockIdx.x / heads, h = blockIdx.x % heads;
  const long long* row = table + (long long)b * 6;
  const unsigned char* kp = (const unsigned char*)row[0] + (long long)h * tokens * 64;
  const float* ks = (const float*)row[1] + h * 128;
  const float* kpad = (const float*)row[2] + h * count;
  const unsigned char* vp = (const unsigned char*)row[3] + (long long)h * tokens * 32;
  const __half* vs = (const __half*)row[4] + (long long)h * tokens * 2;
  const __half* vo = (const __half*)row[5] + (long long)h * tokens * 2;
  if (threadIdx.x < 128) {
    const int r = roles[((long long)b * heads + h) * 128 + threadIdx.x];
    role[threadIdx.x] = r;
    scale[threadIdx.x] = ks[threadIdx.x];
    pad[threadIdx.x] = (r <= -2 && -r - 2 < count) ? kpad[-r - 2] : 0.f;
  }
  __syncthreads();
  const int c0 = (threadIdx.x & 15) * 8;
  int r[8];
  float sc[8], pd[8];
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    r[k] = role[c0 + k];
    sc[k] = scale[c0 + k];
    pd[k] = pad[c0 + k];
  }
  const long long base = (long long)h * stride_h + (position + (long long)b * tokens) * 128;
  const int per_cta = (tokens + gridDim.y - 1) / gridDim.y;
  const int t_begin = blockIdx.y * per_cta, t_end = min(tokens, t_begin + per_cta);
  for (int t = t_begin + (threadIdx.x >> 4); t < t_end; t += 16) {
    const unsigned char* line = kp + (long long)t * 64;
    const unsigned word = *(const unsigned*)(line + (c0 >> 1));
    T vals[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const int slot = (word >> (4 * k)) & 15;
      float value;
      if (r[k] >= 0) {
        const int partner = (line[r[k] >> 1] >> ((r[k] & 1) * 4)) & 15;
        value = (float)(((slot << 4) | partner) - 128) * sc[k];
      } else if (r[k] == -1) {
        value = (float)(slot - 8) * sc[k];
      } else {
        value = pd[k];
      }
      vals[k] = from_float<T>(value);
    }
    *(uint4*)(out_k + base + (long long)t * 128 + c0) = *(const uint4*)vals;
    // values: 8 channels are two bytes of 2-bit codes and share a group of 64
    const unsigned short codes = *(const unsigned short*)(vp + (long long)t * 32 + (c0 >> 2));
    const float vsc = __half2float(vs[t * 2 + (c0 >> 6)]), vof = __half2float(vo[t * 2 + (c0 >> 6)]);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      float value = (float)((codes >> (2 * k)) & 3u) * vsc;
      value = value + vof;
      vals[k] = from_float<T>(value);
    }
    *(uint4*)(out_v + base + (long long)t * 128 + c0) = *(const uint4*)vals;
  }
}

__global__ void build_roles_kernel(const void* salient, const void* donors, int descriptor_i32, int channels, int count,
                                   void* roles, int role_bytes) {
  const long long row = blockIdx.x;
  for (int c = threadIdx.x; c < channels; c += blockDim.x) {
    int role = -1;
    for (int i = 0; i < count; ++i) {
      int s = descriptor_i32 ? ((const int*)salient)[row * count + i] : ((const unsigned char*)salient)[row * count + i];
      int d = descriptor_i32 ? ((const int*)donors)[row * count + i] : ((const unsigned char*)donors)[row * count + i];
      if (s == c) role = d;
      if (d == c) role = -2 - i;
    }
    if (role_bytes == 1)
      ((signed char*)roles)[row * channels + c] = (signed char)role;
    else
      ((short*)roles)[row * channels + c] = (short)role;
  }
}

// ------------------------------------------------------------------------------------------
static bool input_ok(const inq_input_t& in) {
  return in.x && valid_dtype(in.dtype) && in.n_outer >= 1 && in.n_inner >= 1 && in.tokens >= 1 && in.channels >= 1 &&
         in.n_outer * in.n_inner < (1ll << 31);
}

static bool rows_vectorizable(const inq_input_t& in) {
  long long es = dtype_size(in.dtype);
  return in.channels % 8 == 0 && ((uintptr_t)in.x % 16 == 0) && (in.stride_outer * es) % 16 == 0 &&
         (in.stride_inner * es) % 16 == 0 && (in.stride_token * es) % 16 == 0;
}

}  // namespace inq

using namespace inq;

extern "C" int inq_k4_encode(const inq_k4_encode_args_t* a, int32_t* status, inq_stream_t stream_) {
  if (!a || !status || !input_ok(a->in)) return INQ_ERR_ARGUMENT;
  const int C = a->in.channels;
  if (C % 2 || a->count < 0 || a->count > C / 2 || a->sample_stride < 1) return INQ_ERR_ARGUMENT;
  if (C > kMaxChannels) return INQ_ERR_UNSUPPORTED;
  if (!a->payload.base || !a->scales.base || (a->count && !a->padding.base)) return INQ_ERR_ARGUMENT;
  if ((a->salient.base == nullptr) != (a->donors.base == nullptr)) return INQ_ERR_ARGUMENT;
  if (a->roles.base && a->role_bytes != 1 && a->role_bytes != 2) return INQ_ERR_ARGUMENT;
  if (!a->descriptor_i32 && C > 256 && a->salient.base) return INQ_ERR_ARGUMENT;
  K4Params p;
  p.in = make_input(a->in);
  p.sample_stride = a->sample_stride;
  p.count = a->count;
  p.min_error = a->min_error;
  p.payload = make_field(a->payload);
  p.scales = make_field(a->scales);
  p.salient = make_field(a->salient);
  p.donors = make_field(a->donors);
  p.padding = make_field(a->padding);
  p.roles = make_field(a->roles);
  p.descriptor_i32 = a->descriptor_i32;
  p.role_bytes = a->role_bytes;
  p.status = status;
  // 4-byte payload stores need 4-byte aligned rows; the payload row is C/2 bytes.
  p.vector_path = rows_vectorizable(a->in) && ((uintptr_t)a->payload.base % 4 == 0) && a->payload.outer_stride % 4 == 0 &&
                  a->payload.inner_stride % 4 == 0;
  cudaStream_t stream = (cudaStream_t)stream_;
  int threads = ((C + 31) / 32) * 32;
  if (threads < 128 && C % 8 == 0) threads = 128;  // more tokens in flight while packing narrow rows
  size_t shared = k4_shared_bytes(C, a->count, a->in.tokens, a->min_error != 0);
  unsigned grid = (unsigned)(a->in.n_outer * a->in.n_inner);
  if (C == 128 && p.vector_path && a->in.tokens <= kRcpTable && !a->descriptor_i32) {
    const bool regular = a->in.tokens % 8 == 0 && a->sample_stride == 8;
    // whole rows contiguous in memory, in groups of 32 tokens: the shared-memory ring variant
    const bool staged = regular && a->in.tokens % 32 == 0 && a->in.stride_token == C;
    switch (a->in.dtype) {
      case INQ_F32:
        if (regular) k4_encode128_kernel<float, true><<<grid, 128, 0, stream>>>(p);
        else k4_encode128_kernel<float, false><<<grid, 128, 0, stream>>>(p);
        break;
      case INQ_F16:
        if (staged) k4_encode128_kernel<__half, true, true><<<grid, 128, 0, stream>>>(p);
        else if (regular) k4_encode128_kernel<__half, true><<<grid, 128, 0, stream>>>(p);
        else k4_encode128_kernel<__half, false><<<grid, 128, 0, stream>>>(p);
        break;
      default:
        if (staged) k4_encode128_kernel<__nv_bfloat16, true, true><<<grid, 128, 0, stream>>>(p);
        else if (regular) k4_encode128_kernel<__nv_bfloat16, true><<<grid, 128, 0, stream>>>(p);
        else k4_encode128_kernel<__nv_bfloat16, false><<<grid, 128, 0, stream>>>(p);
        break;
    }
  } else if (threads <= 256) {
    switch (a->in.dtype) {
      case INQ_F32: k4_encode_kernel<float, 256><<<grid, threads, shared, stream>>>(p); break;
      case INQ_F16: k4_encode_kernel<__half, 256><<<grid, threads, shared, stream>>>(p); break;
      default: k4_encode_kernel<__nv_bfloat16, 256><<<grid, threads, shared, stream>>>(p); break;
    }
  } else {
    switch (a->in.dtype) {
      case INQ_F32: k4_encode_kernel<float, 1024><<<grid, threads, shared, stream>>>(p); break;
      case INQ_F16: k4_encode_kernel<__half, 1024><<<grid, threads, shared, stream>>>(p); break;
      default: k4_encode_kernel<__nv_bfloat16, 1024><<<grid, threads, shared, stream>>>(p); break;
    }
  }
  INQ_CUDA_CHECK(cudaGetLastError());
  return INQ_OK;
}

extern "C" int inq_k4_statistics(const inq_input_t* in, int32_t sample_stride, float* saliency, float* sampled_mean,
                                 float* donor_error, float* absmax, inq_stream_t stream_) {
  if (!in || !input_ok(*in) || sample_stride < 1) return INQ_ERR_ARGUMENT;
  if (in->channels > kMaxChannels) return INQ_ERR_UNSUPPORTED;
  InputRef ref = make_input(*in);
  cudaStream_t stream = (cudaStream_t)stream_;
  int threads = ((in->channels + 31) / 32) * 32;
  size_t shared = (donor_error && in->tokens <= kRcpTable) ? (size_t)in->tokens * 8 : 0;
  unsigned grid = (unsigned)(in->n_outer * in->n_inner);
  switch (in->dtype) {
    case INQ_F32:
      k4_statistics_kernel<float><<<grid, threads, shared, stream>>>(ref, sample_stride, saliency, sampled_mean, donor_error, absmax);
      break;
    case INQ_F16:
      k4_statistics_kernel<__half><<<grid, threads, shared, stream>>>(ref, sample_stride, saliency, sampled_mean, donor_error, absmax);
      break;
    default:
      k4_statistics_kernel<__nv_bfloat16><<<grid, threads, shared, stream>>>(ref, sample_stride, saliency, sampled_mean, donor_error, absmax);
      break;
  }
  INQ_CUDA_CHECK(cudaGetLastError());
  return INQ_OK;
}

extern "C" int inq_select_donors(const float* saliency, const float* donor_error, int64_t rows, int32_t channels,
                                 int32_t count, int64_t* sources, int64_t* donors, inq_stream_t stream_) {
  if (!saliency || rows < 0 || channels < 1 || count < 0 || count > channels / 2 || rows >= (1ll << 31)) return INQ_ERR_ARGUMENT;
  if (channels > kMaxChannels) return INQ_ERR_UNSUPPORTED;
  if (rows == 0 || count == 0) return INQ_OK;
  if (!sources || !donors) return INQ_ERR_ARGUMENT;
  int threads = ((channels + 31) / 32) * 32;
  size_t shared = (size_t)channels * 12 + kMaxWords * 8 + (size_t)count * 8;
  select_kernel<<<(unsigned)rows, threads, shared, (cudaStream_t)stream_>>>(saliency, donor_error, channels, count,
                                                                             (long long*)sources, (long long*)donors);
  INQ_CUDA_CHECK(cudaGetLastError());
  return INQ_OK;
}

extern "C" int inq_k4_dequantize_strided(const uint8_t* payload, const float* scales, const void* salient, const void* donors,
                                         int32_t descriptor_i32, const float* padding, int64_t rows_outer, int32_t rows_inner,
                                         int32_t tokens, int32_t channels, int32_t count, void* out, int64_t out_stride_outer,
                                         int64_t out_stride_inner, int32_t out_dtype, inq_stream_t stream_) {
  const long long rows = rows_outer * (long long)rows_inner;
  if (!payload || !scales || !out || rows_outer < 1 || rows_inner < 1 || tokens < 1 || channels < 2 || channels % 2 || count < 0 ||
      !valid_dtype(out_dtype) || rows >= (1ll << 31) || out_stride_outer < 0 || out_stride_inner < 0)
    return INQ_ERR_ARGUMENT;
  if (count && (!salient || !donors || !padding)) return INQ_ERR_ARGUMENT;
  if (channels > 4096) return INQ_ERR_UNSUPPORTED;
  cudaStream_t stream = (cudaStream_t)stream_;
  if (channels == 128 && !descriptor_i32 && count <= 64 && out_dtype != INQ_F32 && ((uintptr_t)out % 16) == 0 &&
      out_stride_outer % 8 == 0 && out_stride_inner % 8 == 0 && ((uintptr_t)payload % 4) == 0) {
    // enough CTAs per row to fill the device, at least 64 tokens each
    int split = (int)std::min<long long>((tokens + 63) / 64, std::max<long long>(1, 2048 / rows));
    dim3 fast((unsigned)rows, (unsigned)split);
    if (out_dtype == INQ_F16)
      k4_dequantize128_kernel<__half><<<fast, 256, 0, stream>>>(payload, scales, salient, donors, padding, tokens, count, (__half*)out, rows_inner, out_stride_outer, out_stride_inner);
    else
      k4_dequantize128_kernel<__nv_bfloat16><<<fast, 256, 0, stream>>>(payload, scales, salient, donors, padding, tokens, count, (__nv_bfloat16*)out, rows_inner, out_stride_outer, out_stride_inner);
    INQ_CUDA_CHECK(cudaGetLastError());
    return INQ_OK;
  }
  dim3 grid((unsigned)rows, (unsigned)((tokens + 15) / 16));
  size_t shared = (size_t)channels * 12;
  switch (out_dtype) {
    case INQ_F32:
      k4_dequantize_kernel<float><<<grid, 256, shared, stream>>>(payload, scales, salient, donors, descriptor_i32, padding, tokens, channels, count, (float*)out, rows_inner, out_stride_outer, out_stride_inner);
      break;
    case INQ_F16:
      k4_dequantize_kernel<__half><<<grid, 256, shared, stream>>>(payload, scales, salient, donors, descriptor_i32, padding, tokens, channels, count, (__half*)out, rows_inner, out_stride_outer, out_stride_inner);
      break;
    default:
      k4_dequantize_kernel<__nv_bfloat16><<<grid, 256, shared, stream>>>(payload, scales, salient, donors, descriptor_i32, padding, tokens, channels, count, (__nv_bfloat16*)out, rows_inner, out_stride_outer, out_stride_inner);
      break;
  }
  INQ_CUDA_CHECK(cudaGetLastError());
  return INQ_OK;
}

extern "C" int inq_k4_dequantize(const uint8_t* payload, const float* scales, const void* salient, const void* donors,
                                 int32_t descriptor_i32, const float* padding, int64_t rows, int32_t tokens,
                                 int32_t channels, int32_t count, void* out, int32_t out_dtype, inq_stream_t stream_) {
  return inq_k4_dequantize_strided(payload, scales, salient, donors, descriptor_i32, padding, rows, 1, tokens, channels, count, out,
                                   (int64_t)tokens * channels, 0, out_dtype, stream_);
}

template <typename T>
static int launch_v_encode(const VParams& p, int cpl, dim3 grid, cudaStream_t stream) {
  switch (cpl) {
    case 1: v_encode_kernel<T, 1><<<grid, 256, 0, stream>>>(p); break;
    case 2: v_encode_kernel<T, 2><<<grid, 256, 0, stream>>>(p); break;
    case 4: v_encode_kernel<T, 4><<<grid, 256, 0, stream>>>(p); break;
    case 8: v_encode_kernel<T, 8><<<grid, 256, 0, stream>>>(p); break;
    default: return INQ_ERR_UNSUPPORTED;
  }
  return INQ_OK;
}

extern "C" int inq_v_encode(const inq_v_encode_args_t* a, int32_t* status, inq_stream_t stream_) {
  if (!a || !status || !input_ok(a->in)) return INQ_ERR_ARGUMENT;
  if ((a->bits != 2 && a->bits != 4) || (a->group != 32 && a->group != 64 && a->group != 128)) return INQ_ERR_ARGUMENT;
  const int C = a->in.channels;
  if (C % a->group) return INQ_ERR_ARGUMENT;
  if (!a->payload.base || !a->scales.base || !a->offsets.base) return INQ_ERR_ARGUMENT;
  if (C % 32 || C > 256) return INQ_ERR_UNSUPPORTED;
  VParams p;
  p.in = make_input(a->in);
  p.bits = a->bits;
  p.group = a->group;
  p.payload = make_field(a->payload);
  p.scales = make_field(a->scales);
  p.offsets = make_field(a->offsets);
  p.status = status;
  dim3 grid((unsigned)(a->in.n_outer * a->in.n_inner), (unsigned)((a->in.tokens + 7) / 8));
  cudaStream_t stream = (cudaStream_t)stream_;
  const long long es = dtype_size(a->in.dtype);
  const bool aligned8 = ((uintptr_t)a->in.x % 16 == 0) && (a->in.stride_outer * es) % 16 == 0 &&
                        (a->in.stride_inner * es) % 16 == 0 && (a->in.stride_token * es) % 16 == 0 &&
                        ((uintptr_t)a->payload.base % 4 == 0) && a->payload.outer_stride % 4 == 0 && a->payload.inner_stride % 4 == 0;
  if (C == 128 && aligned8) {
    dim3 fast((unsigned)(a->in.n_outer * a->in.n_inner), (unsigned)((a->in.tokens + 63) / 64));
#define INQ_V128(T)                                                                         \
  if (a->bits == 2) {                                                                       \
    if (a->group == 32) v_encode128_kernel<T, 2, 32><<<fast, 256, 0, stream>>>(p);          \
    else if (a->group == 64) v_encode128_kernel<T, 2, 64><<<fast, 256, 0, stream>>>(p);     \
    else v_encode128_kernel<T, 2, 128><<<fast, 256, 0, stream>>>(p);                        \
  } else {                                                                                  \
    if (a->group == 32) v_encode128_kernel<T, 4, 32><<<fast, 256, 0, stream>>>(p);          \
    else if (a->group == 64) v_encode128_kernel<T, 4, 64><<<fast, 256, 0, stream>>>(p);     \
    else v_encode128_kernel<T, 4, 128><<<fast, 256, 0, stream>>>(p);                        \
  }
    switch (a->in.dtype) {
      case INQ_F32: INQ_V128(float) break;
      case INQ_F16: INQ_V128(__half) break;
      default: INQ_V128(__nv_bfloat16) break;
    }
#undef INQ_V128
    INQ_CUDA_CHECK(cudaGetLastError());
    return INQ_OK;
  }
  int rc;
  switch (a->in.dtype) {
    case INQ_F32: rc = launch_v_encode<float>(p, C / 32, grid, stream); break;
    case INQ_F16: rc = launch_v_encode<__half>(p, C / 32, grid, stream); break;
    default: rc = launch_v_encode<__nv_bfloat16>(p, C / 32, grid, stream); break;
  }
  if (rc != INQ_OK) return rc;
  INQ_CUDA_CHECK(cudaGetLastError());
  return INQ_OK;
}

extern "C" int inq_v_dequantize_strided(const uint8_t* payload, const void* scales, const void* offsets, int64_t rows_outer,
                                        int32_t rows_inner, int32_t tokens, int32_t channels, int32_t bits, int32_t group, void* out,
                                        int64_t out_stride_outer, int64_t out_stride_inner, int32_t out_dtype, inq_stream_t stream_) {
  if (!payload || !scales || !offsets || !out || rows_outer < 1 || rows_inner < 1 || tokens < 1 || (bits != 2 && bits != 4) ||
      (group != 32 && group != 64 && group != 128) || channels % group || !valid_dtype(out_dtype) || out_stride_outer < 0 ||
      out_stride_inner < 0)
    return INQ_ERR_ARGUMENT;
  long long total = rows_outer * (long long)rows_inner * tokens * channels;
  unsigned blocks = (unsigned)((total + 255) / 256);
  cudaStream_t stream = (cudaStream_t)stream_;
  if (channels == 128 && out_dtype != INQ_F32 && ((uintptr_t)out % 16) == 0 && out_stride_outer % 8 == 0 && out_stride_inner % 8 == 0) {
    const long long total_tokens = rows_outer * (long long)rows_inner * tokens;
    const unsigned fast = (unsigned)((total_tokens * 16 + 255) / 256);
    const __half* sc = (const __half*)scales;
    const __half* of = (const __half*)offsets;
    if (out_dtype == INQ_F16 && bits == 2)
      v_dequantize128_kernel<__half, 2><<<fast, 256, 0, stream>>>(payload, sc, of, total_tokens, tokens, group, (__half*)out, rows_inner, out_stride_outer, out_stride_inner);
    else if (out_dtype == INQ_F16)
      v_dequantize128_kernel<__half, 4><<<fast, 256, 0, stream>>>(payload, sc, of, total_tokens, tokens, group, (__half*)out, rows_inner, out_stride_outer, out_stride_inner);
    else if (bits == 2)
      v_dequantize128_kernel<__nv_bfloat16, 2><<<fast, 256, 0, stream>>>(payload, sc, of, total_tokens, tokens, group, (__nv_bfloat16*)out, rows_inner, out_stride_outer, out_stride_inner);
    else
      v_dequantize128_kernel<__nv_bfloat16, 4><<<fast, 256, 0, stream>>>(payload, sc, of, total_tokens, tokens, group, (__nv_bfloat16*)out, rows_inner, out_stride_outer, out_stride_inner);
    INQ_CUDA_CHECK(cudaGetLastError());
    return INQ_OK;
  }
  switch (out_dtype) {
    case INQ_F32:
      v_dequantize_kernel<float><<<blocks, 256, 0, stream>>>(payload, (const __half*)scales, (const __half*)offsets, total, channels, bits, group, (float*)out, tokens, rows_inner, out_stride_outer, out_stride_inner);
      break;
    case INQ_F16:
      v_dequantize_kernel<__half><<<blocks, 256, 0, stream>>>(payload, (const __half*)scales, (const __half*)offsets, total, channels, bits, group, (__half*)out, tokens, rows_inner, out_stride_outer, out_stride_inner);
      break;
    default:
      v_dequantize_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>(payload, (const __half*)scales, (const __half*)offsets, total, channels, bits, group, (__nv_bfloat16*)out, tokens, rows_inner, out_stride_outer, out_stride_inner);
      break;
  }
  INQ_CUDA_CHECK(cudaGetLastError());
  return INQ_OK;
}

extern "C" int inq_v_dequantize(const uint8_t* payload, const void* scales, const void* offsets, int64_t rows,
                                int32_t tokens, int32_t channels, int32_t bits, int32_t group, void* out,
                                int32_t out_dtype, inq_stream_t stream_) {
  return inq_v_dequantize_strided(payload, scales, offsets, rows, 1, tokens, channels, bits, group, out,
                                  (int64_t)tokens * channels, 0, out_dtype, stream_);
}

extern "C" int inq_build_roles(const void* salient, const void* donors, int32_t descriptor_i32, int64_t rows,
                               int32_t channels, int32_t count, void* roles, int32_t role_bytes, inq_stream_t stream_) {
  if (!roles || rows < 0 || channels < 1 || count < 0 || (role_bytes != 1 && role_bytes != 2) || rows >= (1ll << 31))
    return INQ_ERR_ARGUMENT;
  if (count && (!salient || !donors)) return INQ_ERR_ARGUMENT;
  if (rows == 0) return INQ_OK;
  build_roles_kernel<<<(unsigned)rows, 128, 0, (cudaStream_t)stream_>>>(salient, donors, descriptor_i32, channels, count, roles, role_bytes);
  INQ_CUDA_CHECK(cudaGetLastError());
  return INQ_OK;
}

extern "C" int inq_restore_blocks_table(const int64_t* table, const int8_t* roles, int32_t n_blocks, int32_t heads, int32_t tokens,
                                        int32_t count, void* out_key, void* out_value, int64_t stride_h, int64_t position,
                                        int32_t out_dtype, inq_stream_t stream_) {
  if (!table || !roles || !out_key || !out_value || n_blocks < 0 || heads < 1 || tokens < 1 || count < 0 || count > 64)
    return INQ_ERR_ARGUMENT;
  if (out_dtype != INQ_F16 && out_dtype != INQ_BF16) return INQ_ERR_UNSUPPORTED;
  if ((((uintptr_t)out_key | (uintptr_t)out_value) & 15) != 0 || stride_h % 8 != 0 || position < 0) return INQ_ERR_ARGUMENT;
  if (n_blocks == 0) return INQ_OK;
  cudaStream_t stream = (cudaStream_t)stream_;
  // enough CTAs to fill the device when the layer holds few blocks
  const long long rows = (long long)n_blocks * heads;
  int split = 1;
  while (split < 8 && rows * split < 592 && tokens / (split * 2) >= 16) split *= 2;
  const dim3 grid((unsigned)rows, (unsigned)split);
  if (out_dtype == INQ_F16)
    restore_table_kernel<__half><<<grid, 256, 0, stream>>>((const long long*)table, (const signed char*)roles, heads, tokens, count,
                                                          (__half*)out_key, (__half*)out_value, stride_h, position);
  else
    restore_table_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>((const long long*)table, (const signed char*)roles, heads, tokens,
                                                                 count, (__nv_bfloat16*)out_key, (__nv_bfloat16*)out_value, stride_h,
                                                                 position);
  INQ_CUDA_CHECK(cudaGetLastError());
  return INQ_OK;
}
