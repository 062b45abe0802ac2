// Split-KV across the GPUs of one node: exchange of the per-rank partial records over NVLink
// peer memory, fused with their log-sum-exp merge.
//
// Every rank owns an INBOX in its own HBM that all other processes of the node map through CUDA
// IPC.  One launch per decode step and rank does, per chunk of rows (one CTA each):
//   1. push   the chunk of this rank's records is stored straight into every peer's inbox
//             (plain 8-byte stores through the NVLink mapping, no staging copy);
//   2. signal after a system-scope fence, one release store per peer publishes the step number
//             in the flag word (parity, source rank, chunk) of that peer's inbox;
//   3. wait   the CTA polls the flag words of its OWN inbox (local memory) until every peer's
//             chunk of this step has landed -- a bounded wait: it gives up after `spin_limit`
//             polls, reports INQ_STATUS_WAIT_TIMEOUT and returns;
//   4. merge  the log-sum-exp merge of the chunk's rows (the reference's `_reduce_partials`,
//             triton_attention.py:168-181, applied across ranks) writes the final output.
// Chunks are independent, so no grid-wide barrier exists and a chunk is merged as soon as its own
// pieces have arrived.  The inbox is double buffered by step parity: a peer can be at most one
// step ahead of this rank (its next merge needs this rank's next push), so the buffer it writes
// is never the one still being read.
//
// A launch with several ranks (`n_local == world`) runs all of them inside ONE cooperative grid on
// one GPU (blockIdx.y = rank): kernels that wait on one another must not be separate launches
// on a single device.  That form exists to test the protocol without a second GPU.
#include <string.h>

#include "common.cuh"
#include "exchange.cuh"

namespace inq {

constexpr int kExThreads = 256;
constexpr int kExRowPairs = kExRowFloats / 2;     // a row as 8-byte pairs

struct ExchangeRank {
  const float* local;
  unsigned char* inbox[kExMaxWorld];
  void* out;
  int* epoch;      // [0] steps completed, [1] CTAs of the current launch that have finished
  int* status;
  int rank;
};
struct ExchangeParams {
  ExchangeRank ranks[kExMaxWorld];
  int world, rows_per_chunk, spin_limit;
  long long n_rows;
};

__device__ __forceinline__ float ex_exp2(float x) {   // the approximation inq_merge_partials uses
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
template <typename QT>
__global__ void __launch_bounds__(kExThreads, 4) exchange_merge_kernel(const __grid_constant__ ExchangeParams P) {
  const ExchangeRank& R = P.ranks[blockIdx.y];
  const int tid = threadIdx.x, me = R.rank, world = P.world, chunk = blockIdx.x;
  __shared__ int s_failed;
  if (tid == 0) s_failed = 0;
  const int step = R.epoch[0] + 1;
  const int parity = step & 1;
  const long long row0 = (long long)chunk * P.rows_per_chunk;
  const long long row1 = min(row0 + (long long)P.rows_per_chunk, P.n_rows);
  const long long pairs = (row1 - row0) * kExRowPairs;
  const float2* const src = (const float2*)(R.local + row0 * kExRowFloats);

  // 1. push
  for (long long base = 0; base < pairs; base += kExThreads * 4) {
    float2 v[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const long long i = base + j * kExThreads + tid;
      if (i < pairs) v[j] = src[i];
    }
    for (int p = 0; p < world; ++p) {
      if (p == me) continue;
      float2* const dst = (float2*)(ex_data(R.inbox[p], parity, me, world, P.n_rows) + row0 * kExRowFloats);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const long long i = base + j * kExThreads + tid;
        if (i < pairs) dst[i] = v[j];
      }
    }
  }
  // 2. signal
  __threadfence_system();
  __syncthreads();
  if (tid < world && tid != me) st_release_sys(ex_flag(R.inbox[tid], parity, me, chunk), step);
  // 3. wait (bounded)
  if (tid < world && tid != me) {
    const int* const flag = ex_flag(R.inbox[me], parity, tid, chunk);
    int polls = 0;
    while (ld_acquire_sys(flag) - step < 0) {
      if (++polls > P.spin_limit) {
        atomicOr(&s_failed, 1);
        break;
      }
      __nanosleep(100);
    }
  }
  __syncthreads();
  const bool failed = s_failed != 0;
  if (failed && tid == 0) atomicOr(R.status, INQ_STATUS_WAIT_TIMEOUT);

  // 4. merge: one warp per row, four channels per lane; after a failed wait the rows are zeroed
  QT* const out = (QT*)R.out;
  const int warp = tid >> 5, lane = tid & 31;
  for (long long row = row0 + warp; row < row1; row += kExThreads / 32) {
    float o[4] = {0.f, 0.f, 0.f, 0.f}, l = 0.f, top = -1.0e30f;
    if (!failed) {
      for (int p = 0; p < world; ++p) {
        const float* rec = (p == me ? R.local : ex_data(R.inbox[me], parity, p, world, P.n_rows)) + row * kExRowFloats;
        top = fmaxf(top, __ldcg(rec + 128));
      }
      for (int p = 0; p < world; ++p) {
        const float* rec = (p == me ? R.local : ex_data(R.inbox[me], parity, p, world, P.n_rows)) + row * kExRowFloats;
        const float w = ex_exp2(__ldcg(rec + 128) - top);
        const float2 a = __ldcg((const float2*)rec + lane * 2), b = __ldcg((const float2*)rec + lane * 2 + 1);
        o[0] = fmaf(a.x, w, o[0]);
        o[1] = fmaf(a.y, w, o[1]);
        o[2] = fmaf(b.x, w, o[2]);
        o[3] = fmaf(b.y, w, o[3]);
        l = fmaf(__ldcg(rec + 129), w, l);
      }
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) out[row * 128 + lane * 4 + j] = from_float<QT>(failed ? 0.f : o[j] / l);
  }

  // the last CTA of this rank to finish advances the step count for the next launch
  __syncthreads();
  if (tid == 0) {
    const int ticket = atomicAdd(R.epoch + 1, 1);
    if (ticket == (int)gridDim.x - 1) {
      R.epoch[1] = 0;
      __threadfence();
      R.epoch[0] = step;
    }
  }
}

}  // namespace inq

extern "C" int64_t inq_exchange_inbox_bytes(int32_t world, int64_t n_rows) {
  if (world < 1 || world > inq::kExMaxWorld || n_rows < 1) return 0;
  return inq::kExFlagBytes + 2ll * world * n_rows * inq::kExRowFloats * 4;
}

extern "C" int64_t inq_decode_exchange_inbox_bytes(int32_t world, int64_t n_rows) {
  if (world < 1 || world > inq::kExMaxWorld || n_rows < 1) return 0;
  return inq::kExFlagBytes + 2ll * world * n_rows * inq::kExRowFloats * 8;   // every word with its step number
}

extern "C" int inq_exchange_merge(const inq_exchange_args_t* a, inq_stream_t stream_) {
  using namespace inq;
  if (!a || !a->ranks || a->world < 1 || a->world > kExMaxWorld || a->n_rows < 1 || a->n_rows >= (1ll << 31))
    return INQ_ERR_ARGUMENT;
  if (a->n_local != 1 && a->n_local != a->world) return INQ_ERR_ARGUMENT;
  if (a->out_dtype != INQ_F16 && a->out_dtype != INQ_BF16) return INQ_ERR_UNSUPPORTED;
  ExchangeParams P = {};
  for (int i = 0; i < a->n_local; ++i) {
    const inq_exchange_rank_t& r = a->ranks[i];
    if (!r.local || !r.inboxes || !r.out || !r.epoch || !r.status || r.rank < 0 || r.rank >= a->world)
      return INQ_ERR_ARGUMENT;
    if (((uintptr_t)r.local & 7) != 0) return INQ_ERR_ARGUMENT;
    P.ranks[i].local = r.local;
    for (int p = 0; p < a->world; ++p) {
      if (!r.inboxes[p] || ((uintptr_t)r.inboxes[p] & 15) != 0) return INQ_ERR_ARGUMENT;
      P.ranks[i].inbox[p] = (unsigned char*)r.inboxes[p];
    }
    P.ranks[i].out = r.out;
    P.ranks[i].epoch = r.epoch;
    P.ranks[i].status = r.status;
    P.ranks[i].rank = r.rank;
  }
  P.world = a->world;
  P.n_rows = a->n_rows;
  P.spin_limit = a->spin_limit > 0 ? a->spin_limit : kExDefaultSpin;
  // the same cut on every rank: 8 rows per CTA until the CTA count would pass the resident limit
  long long rows_per_chunk = 8;
  if ((a->n_rows + 7) / 8 > kExMaxChunks) rows_per_chunk = ((a->n_rows + kExMaxChunks - 1) / kExMaxChunks + 7) / 8 * 8;
  P.rows_per_chunk = (int)rows_per_chunk;
  const unsigned chunks = (unsigned)((a->n_rows + rows_per_chunk - 1) / rows_per_chunk);

  void (*kernel)(ExchangeParams) = a->out_dtype == INQ_F16 ? exchange_merge_kernel<__half> : exchange_merge_kernel<__nv_bfloat16>;
  int device = 0, sms = 0, per_sm = 0;
  INQ_CUDA_CHECK(cudaGetDevice(&device));
  INQ_CUDA_CHECK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device));
  INQ_CUDA_CHECK(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, kExThreads, 0));
  // CTAs wait for their counterparts on the other ranks: all of a rank's CTAs must be resident
  if ((long long)chunks * a->n_local > (long long)sms * per_sm) return INQ_ERR_CAPACITY;
  cudaStream_t stream = (cudaStream_t)stream_;
  if (a->n_local == 1) {
    kernel<<<dim3(chunks, 1), kExThreads, 0, stream>>>(P);
    INQ_CUDA_CHECK(cudaGetLastError());
  } else {
    void* params[] = {&P};
    INQ_CUDA_CHECK(cudaLaunchCooperativeKernel((const void*)kernel, dim3(chunks, (unsigned)a->n_local), dim3(kExThreads),
                                               params, 0, stream));
  }
  return INQ_OK;
}

// ---------------------------------------------------------------- inbox memory shared over CUDA IPC
extern "C" int inq_peer_buffer_create(int64_t bytes, void** ptr, unsigned char* handle) {
  if (bytes < 1 || !ptr || !handle) return INQ_ERR_ARGUMENT;
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size is part of the ABI");
  void* p = nullptr;
  INQ_CUDA_CHECK(cudaMalloc(&p, (size_t)bytes));
  cudaError_t err = cudaMemset(p, 0, (size_t)bytes);
  if (err == cudaSuccess) err = cudaDeviceSynchronize();
  cudaIpcMemHandle_t h;
  if (err == cudaSuccess) err = cudaIpcGetMemHandle(&h, p);
  if (err != cudaSuccess) {
    cudaFree(p);
    return inq::fail_cuda(err, "inq_peer_buffer_create");
  }
  memcpy(handle, &h, 64);
  *ptr = p;
  return INQ_OK;
}
extern "C" int inq_peer_buffer_open(const unsigned char* handle, void** ptr) {
  if (!handle || !ptr) return INQ_ERR_ARGUMENT;
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, 64);
  INQ_CUDA_CHECK(cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess));
  return INQ_OK;
}
extern "C" int inq_peer_buffer_close(void* ptr) {
  if (!ptr) return INQ_ERR_ARGUMENT;
  INQ_CUDA_CHECK(cudaIpcCloseMemHandle(ptr));
  return INQ_OK;
}
extern "C" int inq_peer_buffer_destroy(void* ptr) {
  if (!ptr) return INQ_ERR_ARGUMENT;
  INQ_CUDA_CHECK(cudaFree(ptr));
  return INQ_OK;
}
