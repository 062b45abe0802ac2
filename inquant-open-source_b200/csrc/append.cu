// Incremental append of one decoded token (all KV heads) into the exact recent tail and,
// while it is still filling, the attention sink.
#include "common.cuh"

#include <algorithm>

namespace inq {

struct AppendParams {
  const uint4* key;
  const uint4* value;
  long long src_stride_h;      // 16-byte units
  uint4* tail_key;
  uint4* tail_value;
  long long tail_stride_h, tail_stride_t;
  int tail_position;
  int* tail_counter;           // optional: position is read here and then incremented
  int tail_capacity;
  uint4* sink_key;
  uint4* sink_value;
  long long sink_stride_h, sink_stride_t;
  int sink_position;           // < 0: the sink is full
  int heads, row_vectors;      // 16-byte vectors per token row
  int* status;
};

// One CTA moves the whole token (heads * row bytes * 2 is a couple of KB), so the device-side
// position can be read, used and advanced without a grid-wide ordering problem.
__device__ __forceinline__ void append_one(const AppendParams& p) {
  __shared__ int s_position;
  if (threadIdx.x == 0) s_position = p.tail_counter ? *p.tail_counter : p.tail_position;
  __syncthreads();
  const int position = s_position;
  if (position < 0 || position >= p.tail_capacity) {
    if (threadIdx.x == 0) atomicOr(p.status, INQ_STATUS_BAD_INDEX);
    return;
  }
  const int total = p.heads * p.row_vectors;
  for (int i = threadIdx.x; i < total; i += blockDim.x) {
    const int h = i / p.row_vectors, v = i % p.row_vectors;
    const uint4 k = p.key[h * p.src_stride_h + v], val = p.value[h * p.src_stride_h + v];
    p.tail_key[h * p.tail_stride_h + position * p.tail_stride_t + v] = k;
    p.tail_value[h * p.tail_stride_h + position * p.tail_stride_t + v] = val;
    if (p.sink_position >= 0) {
      p.sink_key[h * p.sink_stride_h + p.sink_position * p.sink_stride_t + v] = k;
      p.sink_value[h * p.sink_stride_h + p.sink_position * p.sink_stride_t + v] = val;
    }
  }
  if (p.tail_counter && threadIdx.x == 0) *p.tail_counter = position + 1;
}

__global__ void __launch_bounds__(256) append_token_kernel(AppendParams p) { append_one(p); }

// Batched form: CTA i appends the token described by the i-th record of a device array
// (byte strides, as in inq_append_args_t).
__global__ void __launch_bounds__(256) append_batch_kernel(const inq_append_args_t* records, int* status) {
  const inq_append_args_t& a = records[blockIdx.x];
  AppendParams p;
  p.key = (const uint4*)a.key;
  p.value = (const uint4*)a.value;
  p.src_stride_h = a.src_stride_h / 16;
  p.tail_key = (uint4*)a.tail_key;
  p.tail_value = (uint4*)a.tail_value;
  p.tail_stride_h = a.tail_stride_h / 16;
  p.tail_stride_t = a.tail_stride_t / 16;
  p.tail_position = a.tail_position;
  p.tail_counter = a.tail_counter;
  p.tail_capacity = a.tail_capacity;
  p.sink_key = (uint4*)a.sink_key;
  p.sink_value = (uint4*)a.sink_value;
  p.sink_stride_h = a.sink_stride_h / 16;
  p.sink_stride_t = a.sink_stride_t / 16;
  p.sink_position = a.sink_position;
  p.heads = a.heads;
  p.row_vectors = a.row_bytes / 16;
  p.status = status;
  append_one(p);
}

// Row ranges that a sealing update moves (tokens taken by the sink, the remainder that becomes the
// new tail): blockIdx.y picks the copy, the x dimension strides over its 16-byte vectors.
struct RowCopies {
  const uint4* src[4];
  uint4* dst[4];
  long long src_stride_h[4], src_stride_t[4], dst_stride_h[4], dst_stride_t[4];   // 16-byte units
  int tokens[4];
  int heads, row_vectors;
};

__global__ void __launch_bounds__(256) copy_rows_kernel(RowCopies c) {
  const int which = blockIdx.y;
  const int tokens = c.tokens[which];
  const long long total = (long long)c.heads * tokens * c.row_vectors;
  const uint4* src = c.src[which];
  uint4* dst = c.dst[which];
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int v = (int)(i % c.row_vectors);
    const long long row = i / c.row_vectors;
    const int t = (int)(row % tokens), h = (int)(row / tokens);
    dst[h * c.dst_stride_h[which] + t * c.dst_stride_t[which] + v] = src[h * c.src_stride_h[which] + t * c.src_stride_t[which] + v];
  }
}

}  // namespace inq

using namespace inq;

extern "C" int inq_seal_blocks(const inq_seal_args_t* a, int32_t* status, inq_stream_t stream) {
  if (!a || !status || a->n_copies < 0 || a->n_copies > 4) return INQ_ERR_ARGUMENT;
  RowCopies c;
  int n = 0;
  long long most = 0;
  if (a->n_copies) {
    if (a->heads < 1 || a->row_bytes < 16 || a->row_bytes % 16) return INQ_ERR_ARGUMENT;
    for (int i = 0; i < a->n_copies; ++i) {
      const inq_row_copy_t& r = a->copies[i];
      if (r.tokens < 0) return INQ_ERR_ARGUMENT;
      if (!r.tokens) continue;
      if (!r.src || !r.dst || (uintptr_t)r.src % 16 || (uintptr_t)r.dst % 16) return INQ_ERR_ARGUMENT;
      if (r.src_stride_h % 16 || r.src_stride_t % 16 || r.dst_stride_h % 16 || r.dst_stride_t % 16) return INQ_ERR_ARGUMENT;
      c.src[n] = (const uint4*)r.src;
      c.dst[n] = (uint4*)r.dst;
      c.src_stride_h[n] = r.src_stride_h / 16;
      c.src_stride_t[n] = r.src_stride_t / 16;
      c.dst_stride_h[n] = r.dst_stride_h / 16;
      c.dst_stride_t[n] = r.dst_stride_t / 16;
      c.tokens[n] = r.tokens;
      most = std::max(most, (long long)a->heads * r.tokens * (a->row_bytes / 16));
      ++n;
    }
    c.heads = a->heads;
    c.row_vectors = a->row_bytes / 16;
  }
  // every argument is checked before the first launch: a refused call has launched nothing
  int rc;
  if (a->key && (rc = inq_k4_encode(a->key, status, stream)) != INQ_OK) return rc;
  if (a->value_k4 && (rc = inq_k4_encode(a->value_k4, status, stream)) != INQ_OK) return rc;
  if (a->value && (rc = inq_v_encode(a->value, status, stream)) != INQ_OK) return rc;
  if (n) {
    const unsigned blocks = (unsigned)std::min<long long>((most + 255) / 256, 1184);
    copy_rows_kernel<<<dim3(blocks, (unsigned)n), 256, 0, (cudaStream_t)stream>>>(c);
    INQ_CUDA_CHECK(cudaGetLastError());
  }
  return INQ_OK;
}

extern "C" int inq_append_token(const inq_append_args_t* a, inq_stream_t stream) {
  if (!a || !a->key || !a->value || !a->tail_key || !a->tail_value || !a->status) return INQ_ERR_ARGUMENT;
  if (a->heads < 1 || a->row_bytes < 16 || a->row_bytes % 16 || a->tail_capacity < 1) return INQ_ERR_ARGUMENT;
  const int64_t strides[] = {a->src_stride_h, a->tail_stride_h, a->tail_stride_t, a->sink_stride_h, a->sink_stride_t};
  for (int64_t s : strides)
    if (s % 16) return INQ_ERR_ARGUMENT;
  const void* pointers[] = {a->key, a->value, a->tail_key, a->tail_value, a->sink_key, a->sink_value};
  for (const void* ptr : pointers)
    if ((uintptr_t)ptr % 16) return INQ_ERR_ARGUMENT;
  if (a->sink_position >= 0 && (!a->sink_key || !a->sink_value)) return INQ_ERR_ARGUMENT;
  if (!a->tail_counter && (a->tail_position < 0 || a->tail_position >= a->tail_capacity)) return INQ_ERR_ARGUMENT;
  AppendParams p;
  p.key = (const uint4*)a->key;
  p.value = (const uint4*)a->value;
  p.src_stride_h = a->src_stride_h / 16;
  p.tail_key = (uint4*)a->tail_key;
  p.tail_value = (uint4*)a->tail_value;
  p.tail_stride_h = a->tail_stride_h / 16;
  p.tail_stride_t = a->tail_stride_t / 16;
  p.tail_position = a->tail_position;
  p.tail_counter = a->tail_counter;
  p.tail_capacity = a->tail_capacity;
  p.sink_key = (uint4*)a->sink_key;
  p.sink_value = (uint4*)a->sink_value;
  p.sink_stride_h = a->sink_stride_h / 16;
  p.sink_stride_t = a->sink_stride_t / 16;
  p.sink_position = a->sink_position;
  p.heads = a->heads;
  p.row_vectors = a->row_bytes / 16;
  p.status = a->status;
  append_token_kernel<<<1, 256, 0, (cudaStream_t)stream>>>(p);
  INQ_CUDA_CHECK(cudaGetLastError());
  return INQ_OK;
}

extern "C" int inq_append_token_batch(const inq_append_args_t* records_device, int32_t count, int32_t* status,
                                      inq_stream_t stream) {
  if (!records_device || count < 1 || !status) return INQ_ERR_ARGUMENT;
  append_batch_kernel<<<(unsigned)count, 256, 0, (cudaStream_t)stream>>>(records_device, status);
  INQ_CUDA_CHECK(cudaGetLastError());
  return INQ_OK;
}
