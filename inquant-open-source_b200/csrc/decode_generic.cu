// Generic packed decode attention for the codec variants outside the K4/V2 preset: values stored
// as InQuant packed tensors or as 2/4-bit groups of 32, 64 or 128 channels, fp32 / fp16 / bf16
// queries, any even head dimension up to 256, any salient-channel count.  It trades speed for
// coverage: one CTA per (KV head, partition) dequantises 16-token tiles into shared memory the way
// the reference kernel defines them (values rounded to the query dtype before the fp32 dot
// products, triton_attention.py:116-128), keeps fp32 partials (acc, m, l) per query head, and a
// second kernel merges the partitions (triton_attention.py:168-181).  The preset path is
// decode.cu; this file is never on it.
#include <type_traits>

#include "common.cuh"

namespace inq {

constexpr int kGenThreads = 128;
constexpr int kGenTokens = 16;      // tokens per tile
constexpr int kGenHeads = 16;       // query heads per CTA (a KV head's group is cut into such tiles)
constexpr int kGenDense = 64;       // sink / tail tokens per dense partition
constexpr int kGenMaxDim = 256;

struct GenericParams {
  const void* q;
  void* out;
  long long q_sh;
  const long long* table;
  const signed char* key_roles;
  const signed char* value_roles;
  const void *sink_k, *sink_v, *tail_k, *tail_v;
  long long sink_k_sh, sink_k_st, sink_v_sh, sink_v_st, tail_k_sh, tail_k_st, tail_v_sh, tail_v_st;
  int n_blocks, sink_tokens, tail_tokens, sink_parts, tail_parts, n_parts;
  int H, G, T, D, key_pad, value_pad, value_kind, value_bits, value_group;
  float scale_log2e;
  float* partials;    // [Hq][n_parts][D + 2]
};

template <typename QT>
__device__ __forceinline__ float round_to(float v) {
  return to_float<QT>(from_float<QT>(v));
}

// One element of an InQuant-coded block: (block-head row of) payload [T][D/2], scales [D],
// padding [pad], roles [D]; the result is rounded to the query dtype.
template <typename QT>
__device__ __forceinline__ float k4_element(const unsigned char* payload, const float* scales, const float* padding,
                                            const signed char* roles, int D, int tok, int c) {
  const int role = roles[c];
  if (role < -1) return round_to<QT>(padding[-role - 2]);
  const unsigned char* row = payload + (long long)tok * (D / 2);
  const int own = (row[c >> 1] >> (4 * (c & 1))) & 15;
  if (role == -1) return round_to<QT>((float)(own - 8) * scales[c]);
  const int low = (row[role >> 1] >> (4 * (role & 1))) & 15;
  return round_to<QT>((float)(16 * own + low - 128) * scales[c]);
}

template <typename QT>
__global__ void __launch_bounds__(kGenThreads) generic_partials_kernel(const GenericParams P) {
  extern __shared__ float gen_smem[];
  const int D = P.D, tid = threadIdx.x;
  float* qf = gen_smem;                                   // [kGenHeads][D]
  float* kt = qf + kGenHeads * D;                         // [kGenTokens][D + 1]
  float* vt = kt + kGenTokens * (D + 1);                  // [kGenTokens][D + 1]
  float* sc = vt + kGenTokens * (D + 1);                  // [kGenHeads][kGenTokens] scores, then probabilities
  float* alpha = sc + kGenHeads * kGenTokens;             // [kGenHeads]
  float* m_run = alpha + kGenHeads;                       // [kGenHeads]
  float* l_run = m_run + kGenHeads;                       // [kGenHeads]
  const int h = blockIdx.x, part = blockIdx.y, g0 = blockIdx.z * kGenHeads;
  const int g_count = min(kGenHeads, P.G - g0);
  const QT* q = (const QT*)P.q;

  for (int idx = tid; idx < kGenHeads * D; idx += kGenThreads) {
    const int g = idx / D, c = idx % D;
    qf[idx] = g < g_count ? to_float<QT>(q[(long long)(h * P.G + g0 + g) * P.q_sh + c]) * P.scale_log2e : 0.f;
  }
  if (tid < kGenHeads) {
    m_run[tid] = -INFINITY;
    l_run[tid] = 0.f;
  }
  float acc[kGenHeads][2];
#pragma unroll
  for (int g = 0; g < kGenHeads; ++g) acc[g][0] = acc[g][1] = 0.f;

  // what this partition covers
  int tokens;
  const unsigned char *kp = nullptr, *vp = nullptr;
  const float *ks = nullptr, *kpad = nullptr, *vs32 = nullptr, *vpad = nullptr;
  const __half *vs16 = nullptr, *vo16 = nullptr;
  const signed char *kr = nullptr, *vr = nullptr;
  const QT *dk = nullptr, *dv = nullptr;
  long long dk_st = 0, dv_st = 0;
  const bool packed = part < P.n_blocks;
  if (packed) {
    tokens = P.T;
    const long long* row = P.table + (long long)part * 6;
    kp = (const unsigned char*)row[0] + (long long)h * P.T * (D / 2);
    ks = (const float*)row[1] + (long long)h * D;
    kpad = (const float*)row[2] + (long long)h * P.key_pad;
    kr = P.key_roles + ((long long)part * P.H + h) * D;
    if (P.value_kind == 1) {
      vp = (const unsigned char*)row[3] + (long long)h * P.T * (D / 2);
      vs32 = (const float*)row[4] + (long long)h * D;
      vpad = (const float*)row[5] + (long long)h * P.value_pad;
      vr = P.value_roles + ((long long)part * P.H + h) * D;
    } else {
      const int groups = D / P.value_group;
      vp = (const unsigned char*)row[3] + (long long)h * P.T * (D * P.value_bits / 8);
      vs16 = (const __half*)row[4] + (long long)h * P.T * groups;
      vo16 = (const __half*)row[5] + (long long)h * P.T * groups;
    }
  } else {
    const int dp = part - P.n_blocks;
    const bool sink = dp < P.sink_parts;
    const int start = (sink ? dp : dp - P.sink_parts) * kGenDense;
    tokens = min(kGenDense, (sink ? P.sink_tokens : P.tail_tokens) - start);
    dk = (const QT*)(sink ? P.sink_k : P.tail_k) + (long long)h * (sink ? P.sink_k_sh : P.tail_k_sh);
    dv = (const QT*)(sink ? P.sink_v : P.tail_v) + (long long)h * (sink ? P.sink_v_sh : P.tail_v_sh);
    dk_st = sink ? P.sink_k_st : P.tail_k_st;
    dv_st = sink ? P.sink_v_st : P.tail_v_st;
    dk += (long long)start * dk_st;
    dv += (long long)start * dv_st;
  }
  __syncthreads();

  for (int t0 = 0; t0 < tokens; t0 += kGenTokens) {
    const int valid = min(kGenTokens, tokens - t0);
    // ---- keys and values of this tile as the reference's dequantised tensors hold them
    for (int idx = tid; idx < kGenTokens * D; idx += kGenThreads) {
      const int tok = idx / D, c = idx % D;
      float kv = 0.f, vv = 0.f;
      if (tok < valid) {
        const int t = t0 + tok;
        if (packed) {
          kv = k4_element<QT>(kp, ks, kpad, kr, D, t, c);
          if (P.value_kind == 1) {
            vv = k4_element<QT>(vp, vs32, vpad, vr, D, t, c);
          } else {
            const int per_byte = 8 / P.value_bits, groups = D / P.value_group;
            const int byte = vp[(long long)t * (D / per_byte) + c / per_byte];
            const int code = (byte >> ((c % per_byte) * P.value_bits)) & ((1 << P.value_bits) - 1);
            const float s = __half2float(vs16[(long long)t * groups + c / P.value_group]);
            const float o = __half2float(vo16[(long long)t * groups + c / P.value_group]);
            vv = round_to<QT>(__fadd_rn(__fmul_rn((float)code, s), o));
          }
        } else {
          kv = to_float<QT>(dk[(long long)t * dk_st + c]);
          vv = to_float<QT>(dv[(long long)t * dv_st + c]);
        }
      }
      kt[tok * (D + 1) + c] = kv;
      vt[tok * (D + 1) + c] = vv;
    }
    __syncthreads();
    // ---- scores (base 2), two (head, token) pairs per thread
    for (int idx = tid; idx < kGenHeads * kGenTokens; idx += kGenThreads) {
      const int g = idx / kGenTokens, tok = idx % kGenTokens;
      float s = -INFINITY;
      if (g < g_count && tok < valid) {
        s = 0.f;
        const float* qrow = qf + g * D;
        const float* krow = kt + tok * (D + 1);
        for (int c = 0; c < D; ++c) s = fmaf(qrow[c], krow[c], s);
      }
      sc[idx] = s;
    }
    __syncthreads();
    // ---- online softmax per query head; probabilities in the query dtype as the reference feeds them
    if (tid < kGenHeads) {
      const int g = tid;
      float mx = m_run[g];
      for (int tok = 0; tok < kGenTokens; ++tok) mx = fmaxf(mx, sc[g * kGenTokens + tok]);
      const float a = mx == -INFINITY ? 1.f : exp2f(m_run[g] - mx);
      float sum = 0.f;
      for (int tok = 0; tok < kGenTokens; ++tok) {
        const float s = sc[g * kGenTokens + tok];
        const float p = s == -INFINITY ? 0.f : exp2f(s - mx);
        sum += p;
        sc[g * kGenTokens + tok] = round_to<QT>(p);
      }
      alpha[g] = a;
      l_run[g] = l_run[g] * a + sum;
      m_run[g] = mx;
    }
    __syncthreads();
    // ---- accumulate: thread owns channels tid and tid + 128
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int c = tid + half * kGenThreads;
      if (c < D) {
#pragma unroll
        for (int g = 0; g < kGenHeads; ++g) {
          float a = acc[g][half] * alpha[g];
          for (int tok = 0; tok < kGenTokens; ++tok) a = fmaf(sc[g * kGenTokens + tok], vt[tok * (D + 1) + c], a);
          acc[g][half] = a;
        }
      }
    }
    __syncthreads();
  }
  // ---- partial record per query head
#pragma unroll
  for (int g = 0; g < kGenHeads; ++g) {
    if (g < g_count) {
      float* rec = P.partials + ((long long)(h * P.G + g0 + g) * P.n_parts + part) * (D + 2);
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const int c = tid + half * kGenThreads;
        if (c < D) rec[c] = acc[g][half];
      }
      if (tid == 0) {
        rec[D] = m_run[g];
        rec[D + 1] = l_run[g];
      }
    }
  }
}

template <typename QT>
__global__ void __launch_bounds__(kGenMaxDim) generic_reduce_kernel(const float* partials, int n_parts, int D, QT* out) {
  const long long head = blockIdx.x;
  const int c = threadIdx.x;
  const float* base = partials + head * n_parts * (D + 2);
  float top = -INFINITY;
  for (int p = 0; p < n_parts; ++p) top = fmaxf(top, base[(long long)p * (D + 2) + D]);
  float o = 0.f, l = 0.f;
  for (int p = 0; p < n_parts; ++p) {
    const float* rec = base + (long long)p * (D + 2);
    const float m = rec[D];
    const float w = m == -INFINITY ? 0.f : exp2f(m - top);
    if (c < D) o = fmaf(rec[c], w, o);
    l = fmaf(rec[D + 1], w, l);
  }
  if (c < D) out[head * D + c] = from_float<QT>(o / l);
}

template <typename QT>
static int launch_generic(const GenericParams& P, cudaStream_t stream) {
  const int smem = (kGenHeads * P.D + 2 * kGenTokens * (P.D + 1) + kGenHeads * kGenTokens + 3 * kGenHeads) * (int)sizeof(float);
  INQ_CUDA_CHECK(cudaFuncSetAttribute(generic_partials_kernel<QT>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
  const dim3 grid(P.H, P.n_parts, (P.G + kGenHeads - 1) / kGenHeads);
  generic_partials_kernel<QT><<<grid, kGenThreads, smem, stream>>>(P);
  INQ_CUDA_CHECK(cudaGetLastError());
  generic_reduce_kernel<QT><<<P.H * P.G, kGenMaxDim, 0, stream>>>(P.partials, P.n_parts, P.D, (QT*)P.out);
  INQ_CUDA_CHECK(cudaGetLastError());
  return INQ_OK;
}

}  // namespace inq

using namespace inq;

extern "C" int64_t inq_decode_generic_workspace_floats(int32_t q_heads, int32_t n_blocks, int32_t sink_tokens,
                                                       int32_t tail_tokens, int32_t head_dim) {
  const long long parts = (long long)n_blocks + (sink_tokens + kGenDense - 1) / kGenDense + (tail_tokens + kGenDense - 1) / kGenDense;
  return (long long)q_heads * parts * (head_dim + 2);
}

extern "C" int inq_decode_generic(const inq_decode_generic_args_t* a, inq_stream_t stream_) {
  if (!a || !a->q || !a->out || !a->partials) return INQ_ERR_ARGUMENT;
  if (a->kv_heads < 1 || a->q_per_kv < 1 || a->head_dim < 2 || (a->head_dim & 1) || a->head_dim > kGenMaxDim) return INQ_ERR_ARGUMENT;
  if (a->n_blocks < 0 || a->sink_tokens < 0 || a->tail_tokens < 0 || !(a->scale > 0.f)) return INQ_ERR_ARGUMENT;
  if (a->n_blocks + a->sink_tokens + a->tail_tokens == 0) return INQ_ERR_ARGUMENT;
  if (a->n_blocks && (!a->table || !a->key_roles || a->block_tokens < 1)) return INQ_ERR_ARGUMENT;
  if (a->n_blocks && a->value_kind == 1 && !a->value_roles) return INQ_ERR_ARGUMENT;
  if (a->n_blocks && a->value_kind == 0) {
    if ((a->value_bits != 2 && a->value_bits != 4) || a->value_group < 1 || a->head_dim % a->value_group ||
        a->head_dim % (8 / a->value_bits))
      return INQ_ERR_ARGUMENT;
  }
  if (a->value_kind != 0 && a->value_kind != 1) return INQ_ERR_ARGUMENT;
  if ((a->sink_tokens && (!a->sink_key || !a->sink_value)) || (a->tail_tokens && (!a->tail_key || !a->tail_value)))
    return INQ_ERR_ARGUMENT;
  GenericParams P;
  P.q = a->q; P.out = a->out; P.q_sh = a->q_stride_h;
  P.table = (const long long*)a->table; P.key_roles = a->key_roles; P.value_roles = a->value_roles;
  P.sink_k = a->sink_key; P.sink_v = a->sink_value; P.tail_k = a->tail_key; P.tail_v = a->tail_value;
  P.sink_k_sh = a->sink_key_stride_h; P.sink_k_st = a->sink_key_stride_t;
  P.sink_v_sh = a->sink_value_stride_h; P.sink_v_st = a->sink_value_stride_t;
  P.tail_k_sh = a->tail_key_stride_h; P.tail_k_st = a->tail_key_stride_t;
  P.tail_v_sh = a->tail_value_stride_h; P.tail_v_st = a->tail_value_stride_t;
  P.n_blocks = a->n_blocks; P.sink_tokens = a->sink_tokens; P.tail_tokens = a->tail_tokens;
  P.sink_parts = (a->sink_tokens + kGenDense - 1) / kGenDense;
  P.tail_parts = (a->tail_tokens + kGenDense - 1) / kGenDense;
  P.n_parts = P.n_blocks + P.sink_parts + P.tail_parts;
  P.H = a->kv_heads; P.G = a->q_per_kv; P.T = a->block_tokens; P.D = a->head_dim;
  P.key_pad = a->key_pad; P.value_pad = a->value_pad;
  P.value_kind = a->value_kind; P.value_bits = a->value_bits; P.value_group = a->value_group;
  P.scale_log2e = a->scale * 1.4426950408889634f;
  P.partials = a->partials;
  const long long need = (long long)P.H * P.G * P.n_parts * (P.D + 2);
  if (a->partials_floats < need) return INQ_ERR_CAPACITY;
  if (P.n_parts > 65535) return INQ_ERR_CAPACITY;
  cudaStream_t stream = (cudaStream_t)stream_;
  switch (a->dtype) {
    case INQ_F32: return launch_generic<float>(P, stream);
    case INQ_F16: return launch_generic<__half>(P, stream);
    case INQ_BF16: return launch_generic<__nv_bfloat16>(P, stream);
    default: return INQ_ERR_UNSUPPORTED;
  }
}
