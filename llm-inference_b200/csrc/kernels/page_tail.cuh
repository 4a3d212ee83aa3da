// Clearing the unwritten rows of a cache page that a request starts to fill.
//
// Pages pass from request to request without being cleared, and the tensor-core attention kernels
// load whole tiles of a page and mask the rows past a request's last key only in the scores. The
// token that starts a page therefore clears the rows of the page that its step does not fill, in the
// kernel that writes the page.
#pragma once

#include "common.cuh"

// Clears rows `first_row .. page_size` of one (page, kv head) tile, which are contiguous.
template <typename T>
__device__ __forceinline__ void clear_page_tail(T* tile, int first_row, int page_size, int head_dim) {
  if (first_row >= page_size) return;
  const int64_t begin = static_cast<int64_t>(first_row) * head_dim * sizeof(T);
  const int64_t end = static_cast<int64_t>(page_size) * head_dim * sizeof(T);
  unsigned char* base = reinterpret_cast<unsigned char*>(tile);
  if ((static_cast<int64_t>(head_dim) * sizeof(T)) % 16 == 0 && reinterpret_cast<uintptr_t>(base) % 16 == 0) {
    for (int64_t at = begin + threadIdx.x * 16; at < end; at += static_cast<int64_t>(blockDim.x) * 16)
      *reinterpret_cast<uint4*>(base + at) = make_uint4(0u, 0u, 0u, 0u);
  } else {
    T* elems = tile + static_cast<int64_t>(first_row) * head_dim;
    const int count = (page_size - first_row) * head_dim;
    for (int i = threadIdx.x; i < count; i += blockDim.x) elems[i] = from_f32<T>(0.f);
  }
}

// Clears rows `first_row .. page_size` of one (page, kv head) tile, which are contiguous, by one warp.
template <typename T>
__device__ __forceinline__ void clear_page_tail_by_warp(T* tile, int first_row, int page_size, int row_dim, int lane) {
  if (first_row >= page_size) return;
  const int64_t begin = static_cast<int64_t>(first_row) * row_dim * sizeof(T);
  const int64_t end = static_cast<int64_t>(page_size) * row_dim * sizeof(T);
  unsigned char* base = reinterpret_cast<unsigned char*>(tile);
  if ((static_cast<int64_t>(row_dim) * sizeof(T)) % 16 == 0 && reinterpret_cast<uintptr_t>(base) % 16 == 0) {
    for (int64_t at = begin + lane * 16; at < end; at += 32 * 16) *reinterpret_cast<uint4*>(base + at) = make_uint4(0u, 0u, 0u, 0u);
  } else {
    T* elems = tile + static_cast<int64_t>(first_row) * row_dim;
    const int count = (page_size - first_row) * row_dim;
    for (int i = lane; i < count; i += 32) elems[i] = from_f32<T>(0.f);
  }
}
