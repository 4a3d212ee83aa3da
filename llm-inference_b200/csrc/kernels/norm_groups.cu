// Norms that act on a branch's output, a scaled embedding, and the PolyNorm activation.
//
// A "post-norm" layer adds norm(branch(x)) to its residual stream instead of feeding norm(x) to
// the branch:  x <- x + mult * scale[i] * w[i] * d[i] / sqrt(mean_g(d^2) + eps), where d is the
// branch's output and mean_g runs over the consecutive part of the row that holds column i (the
// row is cut into `groups` equal parts, each with a root mean square of its own). The same
// kernel can finish a layer whose stream is a weighted average over depth: with X_0 the
// embedding's output and X_j the stream that left layer j - 1, layer i hands on
// sum_{j <= i + 1} mix[j] * X_j; the X_j live in a history buffer, the newest one still in
// registers. Everything here is 32-bit; `cast` is the stream rounded once to the compute dtype,
// the operand of the next matrix product.
#include "common.cuh"

namespace {

constexpr int kMaxGroups = 64;

// 1 / sqrt(mean(d^2) + eps) of every group of row `d`, by the block's warps (one group per warp
// and turn, lanes stride through it, a fixed tree adds the lanes), into rstd[groups].
template <typename T>
__device__ __forceinline__ void group_rstd(const T* d, int hidden, int groups, float eps, float* rstd) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
  const int size = hidden / groups;
  for (int g = warp; g < groups; g += warps) {
    const T* part = d + g * size;
    float ss = 0.f;
    for (int i = lane; i < size; i += 32) {
      const float v = to_f32<T>(part[i]);
      ss = fmaf(v, v, ss);
    }
    ss = warp_sum(ss);
    if (lane == 0) rstd[g] = 1.f / sqrtf(ss / static_cast<float>(size) + eps);
  }
  __syncthreads();
}

template <typename T>
__global__ void branch_norm_add_kernel(const float* in_x, const T* delta, const float* __restrict__ weight,
                                       const float* __restrict__ scale, float mult, int hidden, int groups, float eps,
                                       float* out_x, float* copy_in, const float* history, int64_t history_stride,
                                       const float* __restrict__ mix, int mix_count, float* mixed_x, T* cast) {
  __shared__ float rstd[kMaxGroups];
  wait_for_predecessor();
  let_successor_start();
  const int64_t row = static_cast<int64_t>(blockIdx.x) * hidden;
  const T* d = delta + row;
  group_rstd<T>(d, hidden, groups, eps, rstd);
  const int size = hidden / groups;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    const float before = in_x[row + i];
    const float normed = to_f32<T>(d[i]) * rstd[i / size] * weight[i];
    const float v = before + mult * (scale ? scale[i] : 1.f) * normed;
    if (copy_in) copy_in[row + i] = before;
    out_x[row + i] = v;
    float next = v;
    if (mix) {
      float acc = 0.f;
      for (int j = 0; j + 1 < mix_count; ++j) acc = fmaf(mix[j], history[j * history_stride + row + i], acc);
      next = fmaf(mix[mix_count - 1], v, acc);
      mixed_x[row + i] = next;
    }
    if (cast) cast[row + i] = from_f32<T>(next);
  }
}

// out[r] = x[rows ? rows[r] : r] normalised in groups, times w; x is the 32-bit stream.
template <typename T>
__global__ void grouped_rmsnorm_kernel(const float* x, const float* __restrict__ weight, const int* rows, int hidden,
                                       int groups, float eps, T* out) {
  __shared__ float rstd[kMaxGroups];
  wait_for_predecessor();
  let_successor_start();
  const int r = rows ? rows[blockIdx.x] : blockIdx.x;
  const float* xr = x + static_cast<int64_t>(r) * hidden;
  group_rstd<float>(xr, hidden, groups, eps, rstd);
  const int size = hidden / groups;
  T* o = out + static_cast<int64_t>(blockIdx.x) * hidden;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) o[i] = from_f32<T>(xr[i] * rstd[i / size] * weight[i]);
}

// x[t] = table[ids[t]] * scale in 32-bit; `cast` (optional) is x rounded to the compute dtype.
template <typename T>
__global__ void embedding_scaled_kernel(const T* __restrict__ table, const int* ids, float scale, float* out, T* cast,
                                        int hidden, int vocab, int* err) {
  wait_for_predecessor();
  let_successor_start();
  const int t = blockIdx.x;
  const int id = ids[t];
  const bool bad = id < 0 || id >= vocab;
  if (bad && threadIdx.x == 0) atomicOr(err, ERRBIT_BAD_TOKEN);
  const T* src = table + static_cast<int64_t>(bad ? 0 : id) * hidden;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    const float v = bad ? 0.f : to_f32<T>(src[i]) * scale;
    out[static_cast<int64_t>(t) * hidden + i] = v;
    if (cast) cast[static_cast<int64_t>(t) * hidden + i] = from_f32<T>(v);
  }
}

// PolyNorm: out = a N(z) + b N(z^2) + c N(z^3) + e, powers element by element, N(y) = y divided by
// the root mean square of the token's row of y (epsilon inside the root). One block per token:
// the three sums of squares (z^2, z^4, z^6) in one pass, the output in a second.
template <typename T>
__global__ void poly_norm_kernel(const T* z, const float* __restrict__ coefficients, int width, float eps, T* out) {
  __shared__ float scratch[32];
  const float a = coefficients[0], b = coefficients[1], c = coefficients[2], e = coefficients[3];
  wait_for_predecessor();
  let_successor_start();
  const T* zr = z + static_cast<int64_t>(blockIdx.x) * width;
  float s1 = 0.f, s2 = 0.f, s3 = 0.f;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    const float v = to_f32<T>(zr[i]);
    const float v2 = v * v;
    s1 += v2;
    s2 = fmaf(v2, v2, s2);
    s3 = fmaf(v2 * v, v2 * v, s3);
  }
  const float n = static_cast<float>(width);
  const float r1 = 1.f / sqrtf(block_sum(s1, scratch) / n + eps);
  const float r2 = 1.f / sqrtf(block_sum(s2, scratch) / n + eps);
  const float r3 = 1.f / sqrtf(block_sum(s3, scratch) / n + eps);
  T* o = out + static_cast<int64_t>(blockIdx.x) * width;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    const float v = to_f32<T>(zr[i]);
    const float v2 = v * v;
    o[i] = from_f32<T>(a * (v * r1) + b * (v2 * r2) + c * (v2 * v * r3) + e);
  }
}

int row_threads(int hidden) { return hidden >= 4096 ? 512 : (hidden >= 1024 ? 256 : 128); }

}  // namespace

B200_API int b200_branch_norm_add(const float* in_x, const void* delta, const float* weight, const float* scale, float mult,
                                  int rows, int hidden, int groups, float eps, float* out_x, float* copy_in,
                                  const float* history, int64_t history_stride, const float* mix, int mix_count,
                                  float* mixed_x, void* cast, int dtype, cudaStream_t stream) {
  if (rows == 0) return 0;
  B200_REQUIRE(rows > 0 && hidden > 0 && groups > 0 && groups <= kMaxGroups && hidden % groups == 0,
               "branch_norm_add: %d columns do not cut into %d groups", hidden, groups);
  B200_REQUIRE(!mix || (mix_count >= 1 && mixed_x && (mix_count == 1 || history)), "branch_norm_add: bad depth mix");
  const int threads = row_threads(hidden);
  if (dtype == DTYPE_F32) {
    launch_kernel(branch_norm_add_kernel<float>, dim3(rows), dim3(threads), 0, stream, in_x, static_cast<const float*>(delta),
                  weight, scale, mult, hidden, groups, eps, out_x, copy_in, history, history_stride, mix, mix_count, mixed_x,
                  static_cast<float*>(cast));
  } else if (dtype == DTYPE_BF16) {
    launch_kernel(branch_norm_add_kernel<__nv_bfloat16>, dim3(rows), dim3(threads), 0, stream, in_x,
                  static_cast<const __nv_bfloat16*>(delta), weight, scale, mult, hidden, groups, eps, out_x, copy_in, history,
                  history_stride, mix, mix_count, mixed_x, static_cast<__nv_bfloat16*>(cast));
  } else {
    return b200_fail("branch_norm_add: unknown dtype %d", dtype);
  }
  return b200_check_launch("branch_norm_add");
}

B200_API int b200_grouped_rmsnorm(const float* x, const float* weight, const int* rows, int num_rows, int hidden, int groups,
                                  float eps, void* out, int dtype, cudaStream_t stream) {
  if (num_rows == 0) return 0;
  B200_REQUIRE(num_rows > 0 && hidden > 0 && groups > 0 && groups <= kMaxGroups && hidden % groups == 0,
               "grouped_rmsnorm: %d columns do not cut into %d groups", hidden, groups);
  const int threads = row_threads(hidden);
  if (dtype == DTYPE_F32) {
    launch_kernel(grouped_rmsnorm_kernel<float>, dim3(num_rows), dim3(threads), 0, stream, x, weight, rows, hidden, groups, eps,
                  static_cast<float*>(out));
  } else if (dtype == DTYPE_BF16) {
    launch_kernel(grouped_rmsnorm_kernel<__nv_bfloat16>, dim3(num_rows), dim3(threads), 0, stream, x, weight, rows, hidden,
                  groups, eps, static_cast<__nv_bfloat16*>(out));
  } else {
    return b200_fail("grouped_rmsnorm: unknown dtype %d", dtype);
  }
  return b200_check_launch("grouped_rmsnorm");
}

B200_API int b200_embedding_scaled(const void* table, const int* ids, float scale, float* out, void* cast, int tokens,
                                   int hidden, int vocab, int dtype, int* err, cudaStream_t stream) {
  if (tokens == 0) return 0;
  B200_REQUIRE(tokens > 0 && hidden > 0 && vocab > 0, "embedding_scaled: bad sizes");
  const int threads = row_threads(hidden);
  if (dtype == DTYPE_F32) {
    launch_kernel(embedding_scaled_kernel<float>, dim3(tokens), dim3(threads), 0, stream, static_cast<const float*>(table), ids,
                  scale, out, static_cast<float*>(cast), hidden, vocab, err);
  } else if (dtype == DTYPE_BF16) {
    launch_kernel(embedding_scaled_kernel<__nv_bfloat16>, dim3(tokens), dim3(threads), 0, stream,
                  static_cast<const __nv_bfloat16*>(table), ids, scale, out, static_cast<__nv_bfloat16*>(cast), hidden, vocab,
                  err);
  } else {
    return b200_fail("embedding_scaled: unknown dtype %d", dtype);
  }
  return b200_check_launch("embedding_scaled");
}

B200_API int b200_poly_norm(const void* z, const float* coefficients, int rows, int width, float eps, void* out, int dtype,
                            cudaStream_t stream) {
  if (rows == 0) return 0;
  B200_REQUIRE(rows > 0 && width > 0, "poly_norm: bad sizes");
  const int threads = row_threads(width);
  if (dtype == DTYPE_F32) {
    launch_kernel(poly_norm_kernel<float>, dim3(rows), dim3(threads), 0, stream, static_cast<const float*>(z), coefficients,
                  width, eps, static_cast<float*>(out));
  } else if (dtype == DTYPE_BF16) {
    launch_kernel(poly_norm_kernel<__nv_bfloat16>, dim3(rows), dim3(threads), 0, stream, static_cast<const __nv_bfloat16*>(z),
                  coefficients, width, eps, static_cast<__nv_bfloat16*>(out));
  } else {
    return b200_fail("poly_norm: unknown dtype %d", dtype);
  }
  return b200_check_launch("poly_norm");
}
