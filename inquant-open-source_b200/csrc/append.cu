// Incremental append of one decoded token (all KV heads) into the exact recent tail and,
// while it is still filling, the attention sink.
#include "common.cuh"

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

}  // namespace inq

using namespace inq;

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
