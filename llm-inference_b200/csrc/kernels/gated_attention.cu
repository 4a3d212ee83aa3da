// What surrounds the paged attention kernels in a mixer without position encoding: unit-RMS queries
// and keys, values blended with an earlier layer's values of the same token, the cache write, and a
// gate per head on the way out.
//
// `norm_kv_write`: per new token, every query and key head is divided by its root mean square over
// its `dim` numbers (no weight; eps inside the root), all in 32-bit; values become
// (1 - l) v + l v_first when the layer blends (`v_first` [tokens][kv_heads * vdim], `l` one number on the
// device), or are stored into `v_first` when the layer is the one the others blend with. Queries go to
// a dense buffer and keys and values into the token's page; rows are `row_dim` wide in all three
// (`row_dim` >= dim, vdim: the arena has one row width for keys and values), the rest zero, which
// changes neither a score nor the part of the output that is read. The token that starts a page
// clears the rows its step does not fill.
//
// `head_gate`: out[t][h][:vdim] = attn[t][h][:vdim] * sigmoid(gate[t][h]).
#include "common.cuh"
#include "page_tail.cuh"

namespace {

// One warp per (token, head): query heads first, then key heads, then value heads. `proj` rows hold
// [q (q_heads*dim) | k (kv_heads*dim) | v (kv_heads*vdim) | ...], `ld` numbers apart.
template <typename T>
__global__ void norm_kv_write_kernel(const T* proj, int ld, const int* __restrict__ positions, const int* __restrict__ token_seq,
                                     const int* __restrict__ seq_kv_len, const int* __restrict__ block_table, int max_pages,
                                     int num_pages, T* k_arena, T* v_arena, T* q_out, T* v_first, const float* blend, int blend_mode,
                                     int tokens, int q_heads, int kv_heads, int dim, int vdim, int row_dim, int page_size,
                                     int normalise, float eps, int write_kv, int* err) {
  let_successor_start();
  const int lane = threadIdx.x & 31;
  const int heads_all = q_heads + 2 * kv_heads;
  const int64_t item = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const bool live = item < static_cast<int64_t>(tokens) * heads_all;
  const int t = live ? static_cast<int>(item / heads_all) : 0, head = live ? static_cast<int>(item % heads_all) : 0;
  const bool is_q = head < q_heads, is_k = !is_q && head < q_heads + kv_heads;
  const int pos = positions[t];
  T* dst = nullptr;
  int clear_from = 0;
  if (!live) {
  } else if (is_q) {
    dst = q_out + (static_cast<int64_t>(t) * q_heads + head) * row_dim;
  } else if (write_kv) {
    const int logical = pos / page_size;
    if (pos < 0 || logical >= max_pages) {
      if (lane == 0) atomicOr(err, ERRBIT_BAD_POSITION);
    } else {
      const int page = block_table[static_cast<int64_t>(token_seq[t]) * max_pages + logical];
      if (page < 0 || page >= num_pages) {
        if (lane == 0) atomicOr(err, ERRBIT_BAD_PAGE);
      } else {
        const int kv_head = is_k ? head - q_heads : head - q_heads - kv_heads;
        dst = (is_k ? k_arena : v_arena) + kv_row_offset(page, kv_head, pos % page_size, kv_heads, page_size, row_dim);
        if (pos % page_size == 0 && seq_kv_len != nullptr) clear_from = max(1, seq_kv_len[token_seq[t]] - pos);
      }
    }
  }
  wait_for_predecessor();
  if (!live) return;
  const T* row = proj + static_cast<int64_t>(t) * ld;
  if (dst != nullptr && clear_from > 0) clear_page_tail_by_warp(dst, clear_from, page_size, row_dim, lane);
  if (is_q || is_k) {
    if (dst == nullptr) return;
    const T* src = row + (is_q ? head * dim : q_heads * dim + (head - q_heads) * dim);
    float inv = 1.f;
    if (normalise) {
      float ss = 0.f;
      for (int i = lane; i < dim; i += 32) {
        const float x = to_f32<T>(src[i]);
        ss = fmaf(x, x, ss);
      }
      ss = warp_sum(ss);
      inv = 1.f / sqrtf(ss / static_cast<float>(dim) + eps);
    }
    for (int i = lane; i < row_dim; i += 32) dst[i] = from_f32<T>(i < dim ? to_f32<T>(src[i]) * inv : 0.f);
    return;
  }
  // a value head: blend or publish, then store
  const int kv_head = head - q_heads - kv_heads;
  const T* src = row + (q_heads + kv_heads) * dim + kv_head * vdim;
  T* shared_row = v_first ? v_first + (static_cast<int64_t>(t) * kv_heads + kv_head) * vdim : nullptr;
  const float lam = blend_mode == 2 ? *blend : 0.f;
  for (int i = lane; i < row_dim; i += 32) {
    float x = 0.f;
    if (i < vdim) {
      x = to_f32<T>(src[i]);
      if (blend_mode == 1) shared_row[i] = src[i];
      else if (blend_mode == 2) x = fmaf(lam, to_f32<T>(shared_row[i]), (1.f - lam) * x);
    }
    if (dst != nullptr) dst[i] = from_f32<T>(x);
  }
}

// attn rows are [heads][row_dim]; gate logits sit at proj[t * ld + gate_offset + h].
template <typename T>
__global__ void head_gate_kernel(const T* attn, const T* proj, int ld, int gate_offset, int tokens, int heads, int vdim, int row_dim,
                                 T* out) {
  wait_for_predecessor();
  let_successor_start();
  const int64_t total = static_cast<int64_t>(tokens) * heads * vdim;
  for (int64_t idx = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; idx < total; idx += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int i = static_cast<int>(idx % vdim);
    const int64_t th = idx / vdim;
    const int h = static_cast<int>(th % heads);
    const int64_t t = th / heads;
    const float g = proj ? 1.f / (1.f + expf(-to_f32<T>(proj[t * ld + gate_offset + h]))) : 1.f;
    out[idx] = from_f32<T>(to_f32<T>(attn[th * row_dim + i]) * g);
  }
}

// The same for bfloat16 when heads are not padded and hold a multiple of eight numbers: eight a thread.
__global__ void head_gate_wide_kernel(const __nv_bfloat16* attn, const __nv_bfloat16* proj, int ld, int gate_offset, int tokens, int heads,
                                      int vdim, __nv_bfloat16* out) {
  wait_for_predecessor();
  let_successor_start();
  const int chunks = vdim / 8;
  const int64_t total = static_cast<int64_t>(tokens) * heads * chunks;
  for (int64_t idx = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; idx < total; idx += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t th = idx / chunks;
    const int h = static_cast<int>(th % heads);
    const int64_t t = th / heads;
    const float g = proj ? 1.f / (1.f + expf(-__bfloat162float(proj[t * ld + gate_offset + h]))) : 1.f;
    const uint4 raw = *reinterpret_cast<const uint4*>(attn + idx * 8);
    const __nv_bfloat162* a2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
    uint4 packed;
    __nv_bfloat162* y2 = reinterpret_cast<__nv_bfloat162*>(&packed);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 a = __bfloat1622float2(a2[j]);
      y2[j] = __floats2bfloat162_rn(a.x * g, a.y * g);
    }
    *reinterpret_cast<uint4*>(out + idx * 8) = packed;
  }
}

}  // namespace

B200_API int b200_norm_kv_write(const void* proj, int ld, const int* positions, const int* token_seq, const int* seq_kv_len,
                                const int* block_table, int max_pages, int num_pages, void* k_arena, void* v_arena, void* q_out,
                                void* v_first, const float* blend, int blend_mode, int tokens, int q_heads, int kv_heads, int dim,
                                int vdim, int row_dim, int page_size, int normalise, float eps, int write_kv, int dtype, int* err,
                                cudaStream_t stream) {
  if (tokens == 0) return 0;
  B200_REQUIRE(tokens > 0 && q_heads > 0 && kv_heads > 0 && dim > 0 && vdim > 0 && row_dim >= dim && row_dim >= vdim,
               "norm_kv_write: bad sizes");
  B200_REQUIRE(ld >= q_heads * dim + kv_heads * (dim + vdim), "norm_kv_write: rows of %d numbers do not hold the projections", ld);
  B200_REQUIRE(blend_mode >= 0 && blend_mode <= 2 && (blend_mode == 0 || v_first != nullptr) && (blend_mode != 2 || blend != nullptr),
               "norm_kv_write: a blending layer needs the shared values and its factor");
  // Four warps a block for prompt portions; a warp a block for short steps, so that they spread over the SMs.
  const int64_t items = static_cast<int64_t>(tokens) * (q_heads + 2 * kv_heads);
  const int warps = items >= 2048 ? 4 : 1;
  const int threads = 32 * warps;
  const dim3 grid(static_cast<unsigned>((items + warps - 1) / warps));
  if (dtype == DTYPE_F32) {
    launch_kernel(norm_kv_write_kernel<float>, grid, dim3(threads), 0, stream, static_cast<const float*>(proj), ld, positions, token_seq,
                  seq_kv_len, block_table, max_pages, num_pages, static_cast<float*>(k_arena), static_cast<float*>(v_arena),
                  static_cast<float*>(q_out), static_cast<float*>(v_first), blend, blend_mode, tokens, q_heads, kv_heads, dim, vdim,
                  row_dim, page_size, normalise, eps, write_kv, err);
  } else if (dtype == DTYPE_BF16) {
    launch_kernel(norm_kv_write_kernel<__nv_bfloat16>, grid, dim3(threads), 0, stream, static_cast<const __nv_bfloat16*>(proj), ld,
                  positions, token_seq, seq_kv_len, block_table, max_pages, num_pages, static_cast<__nv_bfloat16*>(k_arena),
                  static_cast<__nv_bfloat16*>(v_arena), static_cast<__nv_bfloat16*>(q_out), static_cast<__nv_bfloat16*>(v_first), blend,
                  blend_mode, tokens, q_heads, kv_heads, dim, vdim, row_dim, page_size, normalise, eps, write_kv, err);
  } else {
    return b200_fail("norm_kv_write: unknown dtype %d", dtype);
  }
  return b200_check_launch("norm_kv_write");
}

B200_API int b200_head_gate(const void* attn, const void* proj, int ld, int gate_offset, int tokens, int heads, int vdim, int row_dim,
                            void* out, int dtype, cudaStream_t stream) {
  if (tokens == 0) return 0;
  B200_REQUIRE(tokens > 0 && heads > 0 && vdim > 0 && row_dim >= vdim, "head_gate: bad sizes");
  const int threads = 256;
  const int64_t total = static_cast<int64_t>(tokens) * heads * vdim;
  const int64_t want = (total + threads - 1) / threads;
  const dim3 grid(static_cast<unsigned>(want < 65535 ? want : 65535));
  if (dtype == DTYPE_F32) {
    launch_kernel(head_gate_kernel<float>, grid, dim3(threads), 0, stream, static_cast<const float*>(attn), static_cast<const float*>(proj),
                  ld, gate_offset, tokens, heads, vdim, row_dim, static_cast<float*>(out));
  } else if (dtype == DTYPE_BF16 && row_dim == vdim && vdim % 8 == 0 && reinterpret_cast<uintptr_t>(attn) % 16 == 0 &&
             reinterpret_cast<uintptr_t>(out) % 16 == 0) {
    const int64_t wide = (total / 8 + threads - 1) / threads;
    launch_kernel(head_gate_wide_kernel, dim3(static_cast<unsigned>(wide < 65535 ? wide : 65535)), dim3(threads), 0, stream,
                  static_cast<const __nv_bfloat16*>(attn), static_cast<const __nv_bfloat16*>(proj), ld, gate_offset, tokens, heads, vdim,
                  static_cast<__nv_bfloat16*>(out));
  } else if (dtype == DTYPE_BF16) {
    launch_kernel(head_gate_kernel<__nv_bfloat16>, grid, dim3(threads), 0, stream, static_cast<const __nv_bfloat16*>(attn),
                  static_cast<const __nv_bfloat16*>(proj), ld, gate_offset, tokens, heads, vdim, row_dim, static_cast<__nv_bfloat16*>(out));
  } else {
    return b200_fail("head_gate: unknown dtype %d", dtype);
  }
  return b200_check_launch("head_gate");
}
