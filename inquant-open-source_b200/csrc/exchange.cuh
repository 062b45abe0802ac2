// Layout of a split-KV inbox and the system-scope accesses of its flag words, shared by the
// stand-alone exchange kernel and by the decode kernel's own exchange of a pair's record.
//
// Inbox of one rank: flag words [parity][source rank][chunk] (the step number a source has
// published for that chunk), then records [parity][source rank][row][130 floats]
// (acc[128], m in base-2 units, l).  Double buffered by step parity: a peer can be at most one step
// ahead of the rank that owns the inbox (its next merge needs that rank's next records).
#pragma once

namespace inq {

constexpr int kExMaxWorld = 8;
constexpr int kExMaxChunks = 512;                 // flag words per source rank and parity
constexpr int kExRowFloats = 130;                 // acc[128], m (base-2 units), l
constexpr long long kExFlagBytes = 2ll * kExMaxWorld * kExMaxChunks * 4;   // [parity][src][chunk]
constexpr int kExDefaultSpin = 1 << 21;           // polls of >= 100 ns: gives up after a fraction of a second

__device__ __forceinline__ void st_release_sys(int* p, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ int* ex_flag(unsigned char* inbox, int parity, int src, int chunk) {
  return (int*)inbox + ((long long)parity * kExMaxWorld + src) * kExMaxChunks + chunk;
}
__device__ __forceinline__ float* ex_data(unsigned char* inbox, int parity, int src, int world, long long n_rows) {
  return (float*)(inbox + kExFlagBytes) + ((long long)parity * world + src) * n_rows * kExRowFloats;
}
// The decode kernel's own exchange keeps the same record grid but every 32-bit word of a record is
// an 8-byte pair {word, step number it belongs to}; it uses no flag words.
__device__ __forceinline__ uint2* ex_tagged(unsigned char* inbox, int parity, int src, int world, long long n_rows) {
  return (uint2*)(inbox + kExFlagBytes) + ((long long)parity * world + src) * n_rows * kExRowFloats;
}

}  // namespace inq
