// Scatter of already-encoded codec output into physical pages of the serving layout, one launch
// (reference: extensions/vllm/src/inquant_vllm/packing.py:7-55 `_write_pages` / `write_codec_pages`).
// One CTA per (page, KV head): 16-byte copies of the head's slice of every field, and the int16
// role map of the page built from the descriptor lists on the way.
#include "common.cuh"

namespace inq {

struct WritePagesParams {
  const unsigned char* key_payload;
  const unsigned char* key_scales;
  const unsigned char* salient;
  const unsigned char* donors;
  const unsigned char* key_padding;
  const unsigned char* value_payload;
  const unsigned char* value_scales;
  const unsigned char* value_offsets;
  long long pages;
  int heads, block_tokens, count;
  unsigned char* pool;
  long long page_bytes, num_slots;
  long long off_ks, off_km, off_kp, off_vp, off_vs, off_vo;
  const void* page_ids;
  int page_ids_i64;
  int* status;
};

__device__ __forceinline__ void copy16(unsigned char* dst, const unsigned char* src, int bytes) {
  for (int i = threadIdx.x * 16; i < bytes; i += blockDim.x * 16) *(uint4*)(dst + i) = *(const uint4*)(src + i);
}

__global__ void __launch_bounds__(256) write_pages_kernel(const WritePagesParams p) {
  const long long page = blockIdx.x / p.heads;
  const int h = (int)(blockIdx.x % p.heads);
  const long long slot = p.page_ids_i64 ? ((const long long*)p.page_ids)[page] : (long long)((const int*)p.page_ids)[page];
  if (p.num_slots > 0 && (slot < 0 || slot >= p.num_slots)) {   // uniform over the CTA: the page is not written
    if (threadIdx.x == 0) atomicOr(p.status, INQ_STATUS_BAD_INDEX);
    return;
  }
  unsigned char* const out = p.pool + slot * p.page_bytes;
  const long long row = page * p.heads + h;
  const int B = p.block_tokens;
  copy16(out + (long long)h * B * 64, p.key_payload + row * B * 64, B * 64);
  copy16(out + p.off_ks + h * 512, p.key_scales + row * 512, 512);
  copy16(out + p.off_kp + h * 64, p.key_padding + row * 64, 64);
  copy16(out + p.off_vp + (long long)h * B * 32, p.value_payload + row * B * 32, B * 32);
  copy16(out + p.off_vs + (long long)h * B * 4, p.value_scales + row * B * 4, B * 4);
  copy16(out + p.off_vo + (long long)h * B * 4, p.value_offsets + row * B * 4, B * 4);
  // role map: donor channel for a salient channel, -1 for a normal one, -2 - i for the i-th donor
  __shared__ __align__(16) short roles[128];
  if (threadIdx.x < 128) roles[threadIdx.x] = -1;
  __syncthreads();
  if ((int)threadIdx.x < p.count) {
    const int i = threadIdx.x;
    const int source = p.salient[row * p.count + i], donor = p.donors[row * p.count + i];
    if (source < 128 && donor < 128) {
      roles[source] = (short)donor;
      roles[donor] = (short)(-2 - i);
    } else {
      atomicOr(p.status, INQ_STATUS_BAD_INDEX);
    }
  }
  __syncthreads();
  if (threadIdx.x < 16) *(uint4*)(out + p.off_km + h * 256 + threadIdx.x * 16) = *(const uint4*)((const unsigned char*)roles + threadIdx.x * 16);
}

}  // namespace inq

extern "C" int inq_write_codec_pages(const inq_write_pages_args_t* a, inq_stream_t stream) {
  if (!a || !a->key_payload || !a->key_scales || !a->key_padding || !a->value_payload || !a->value_scales || !a->value_offsets)
    return INQ_ERR_ARGUMENT;
  if (!a->pool || !a->page_ids || !a->status || a->pages < 0 || a->heads < 1 || a->page_bytes < 1) return INQ_ERR_ARGUMENT;
  if (a->block_tokens < 4 || a->block_tokens % 4 || a->count < 0 || a->count > 64 || (a->count && (!a->salient || !a->donors)))
    return INQ_ERR_ARGUMENT;
  if (a->count != 16) return INQ_ERR_UNSUPPORTED;   // the page layout holds 16 padding values per head
  const uintptr_t bits = (uintptr_t)a->key_payload | (uintptr_t)a->key_scales | (uintptr_t)a->key_padding | (uintptr_t)a->value_payload |
                         (uintptr_t)a->value_scales | (uintptr_t)a->value_offsets | (uintptr_t)a->pool | (uintptr_t)a->page_bytes;
  for (int i = 0; i < 6; ++i)
    if (a->page_offsets[i] % 16) return INQ_ERR_ARGUMENT;
  if (bits % 16) return INQ_ERR_ARGUMENT;
  if (a->pages == 0) return INQ_OK;
  if (a->pages * a->heads >= (1ll << 31)) return INQ_ERR_UNSUPPORTED;
  inq::WritePagesParams p;
  p.key_payload = (const unsigned char*)a->key_payload; p.key_scales = (const unsigned char*)a->key_scales;
  p.salient = (const unsigned char*)a->salient; p.donors = (const unsigned char*)a->donors;
  p.key_padding = (const unsigned char*)a->key_padding; p.value_payload = (const unsigned char*)a->value_payload;
  p.value_scales = (const unsigned char*)a->value_scales; p.value_offsets = (const unsigned char*)a->value_offsets;
  p.pages = a->pages; p.heads = a->heads; p.block_tokens = a->block_tokens; p.count = a->count;
  p.pool = (unsigned char*)a->pool; p.page_bytes = a->page_bytes; p.num_slots = a->num_slots;
  p.off_ks = a->page_offsets[0]; p.off_km = a->page_offsets[1]; p.off_kp = a->page_offsets[2];
  p.off_vp = a->page_offsets[3]; p.off_vs = a->page_offsets[4]; p.off_vo = a->page_offsets[5];
  p.page_ids = a->page_ids; p.page_ids_i64 = a->page_ids_i64; p.status = a->status;
  inq::write_pages_kernel<<<(unsigned)(a->pages * a->heads), 256, 0, (cudaStream_t)stream>>>(p);
  INQ_CUDA_CHECK(cudaGetLastError());
  return INQ_OK;
}
