// Several residual streams per token (hyper-connections), the embedding that fills them, and the
// soft cap on logits.
//
// A token carries n streams x_1 .. x_n of the model's width (32-bit, laid out [tokens][n][width]).
// A sublayer reads u = sum_s a[s] x_s through an RMS norm, and its output y goes back into all
// streams at once: x_t <- sum_s M[s][t] x_s + b[t] y. Here the write of one sublayer and the read
// and norm of the next are one kernel (`hyper_norm`): per column it loads the n old values, forms
// the n new ones, stores them, and keeps u in shared memory until the row's sum of squares is
// known. With n = 1, a = b = M = 1 this is the ordinary "add the branch, then RMS-norm" kernel.
// The model's last norm is the same kernel with a = 1 (the sum of the streams) on gathered rows.
//
// Embedding: x = table[token] * scale + e(p), e(p)[2i] = sin(p f_i), e(p)[2i+1] = cos(p f_i), with
// the f_i tabulated by the host; the angle and its sine and cosine are 32-bit.
#include "common.cuh"

namespace {

constexpr int kMaxStreams = 8;

template <typename T>
__global__ void embedding_sinusoid_kernel(const T* __restrict__ table, const int* ids, const int* __restrict__ positions,
                                          const float* __restrict__ inv_freq, float scale, float* out, int streams, int hidden,
                                          int vocab, int* err) {
  wait_for_predecessor();
  let_successor_start();
  const int t = blockIdx.x;
  const int id = ids[t];
  float* dst = out + static_cast<int64_t>(t) * streams * hidden;
  const bool bad = id < 0 || id >= vocab;
  if (bad && threadIdx.x == 0) atomicOr(err, ERRBIT_BAD_TOKEN);
  const T* src = table + static_cast<int64_t>(bad ? 0 : id) * hidden;
  const float pos = static_cast<float>(positions[t]);
  for (int i = threadIdx.x; i < hidden / 2; i += blockDim.x) {
    float sn, cs;
    sincosf(pos * inv_freq[i], &sn, &cs);
    const float e0 = bad ? 0.f : fmaf(to_f32<T>(src[2 * i]), scale, sn);
    const float e1 = bad ? 0.f : fmaf(to_f32<T>(src[2 * i + 1]), scale, cs);
    for (int s = 0; s < streams; ++s) {
      dst[s * hidden + 2 * i] = e0;
      dst[s * hidden + 2 * i + 1] = e1;
    }
  }
}

// One block per output row. `y` (may be null): the pending branch output of the sublayer in
// front, written into the streams with `mix_w` [n][n] (indexed [from][to]) and `out_w` [n]; the new
// streams are stored back unless rows are gathered. `in_w` (null: ones) weighs the streams into u.
template <typename T, int N>
__global__ void hyper_norm_kernel(float* x, const T* y, const float* __restrict__ mix_w, const float* __restrict__ out_w,
                                  const float* __restrict__ in_w, const float* __restrict__ weight, const int* rows, int hidden,
                                  float eps, T* out) {
  extern __shared__ float u_row[];  // [hidden]
  __shared__ float scratch[32];
  float m[N][N], b[N], a[N];
#pragma unroll
  for (int s = 0; s < N; ++s) {
    a[s] = in_w ? in_w[s] : 1.f;
    b[s] = y ? out_w[s] : 0.f;
#pragma unroll
    for (int r = 0; r < N; ++r) m[s][r] = y ? mix_w[s * N + r] : (s == r ? 1.f : 0.f);
  }
  wait_for_predecessor();
  let_successor_start();
  const int row = rows ? rows[blockIdx.x] : blockIdx.x;
  float* xr = x + static_cast<int64_t>(row) * N * hidden;
  const T* yr = y ? y + static_cast<int64_t>(row) * hidden : nullptr;
  float ss = 0.f;
  for (int d = threadIdx.x; d < hidden; d += blockDim.x) {
    float old[N], fresh[N];
#pragma unroll
    for (int s = 0; s < N; ++s) old[s] = xr[s * hidden + d];
    float u = 0.f;
    if (yr) {
      const float yd = to_f32<T>(yr[d]);
#pragma unroll
      for (int r = 0; r < N; ++r) {
        float v = b[r] * yd;
#pragma unroll
        for (int s = 0; s < N; ++s) v = fmaf(m[s][r], old[s], v);
        fresh[r] = v;
      }
      if (!rows) {
#pragma unroll
        for (int r = 0; r < N; ++r) xr[r * hidden + d] = fresh[r];
      }
    } else {
#pragma unroll
      for (int r = 0; r < N; ++r) fresh[r] = old[r];
    }
#pragma unroll
    for (int r = 0; r < N; ++r) u = fmaf(a[r], fresh[r], u);
    u_row[d] = u;
    ss = fmaf(u, u, ss);
  }
  const float total = block_sum(ss, scratch);
  const float inv = 1.f / sqrtf(total / static_cast<float>(hidden) + eps);
  T* dst = out + static_cast<int64_t>(blockIdx.x) * hidden;
  for (int d = threadIdx.x; d < hidden; d += blockDim.x) dst[d] = from_f32<T>(u_row[d] * inv * weight[d]);
}

__global__ void softcap_kernel(float* logits, int64_t count, float cap) {
  wait_for_predecessor();
  let_successor_start();
  const float inv = 1.f / cap;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < count; i += static_cast<int64_t>(gridDim.x) * blockDim.x)
    logits[i] = cap * tanhf(logits[i] * inv);
}

template <typename T, int N>
int launch_hyper_norm(float* x, const void* y, const float* mix_w, const float* out_w, const float* in_w, const float* weight,
                      const int* rows, int count, int hidden, float eps, void* out, cudaStream_t stream) {
  const size_t smem = sizeof(float) * hidden;
  if (smem > 48 * 1024) cudaFuncSetAttribute(hyper_norm_kernel<T, N>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
  const int threads = hidden >= 2048 ? 512 : (hidden >= 512 ? 256 : 128);
  launch_kernel(hyper_norm_kernel<T, N>, dim3(count), dim3(threads), smem, stream, x, static_cast<const T*>(y), mix_w, out_w, in_w,
                weight, rows, hidden, eps, static_cast<T*>(out));
  return b200_check_launch("hyper_norm");
}

template <typename T>
int dispatch_hyper_norm(int streams, float* x, const void* y, const float* mix_w, const float* out_w, const float* in_w,
                        const float* weight, const int* rows, int count, int hidden, float eps, void* out, cudaStream_t stream) {
  switch (streams) {
    case 1: return launch_hyper_norm<T, 1>(x, y, mix_w, out_w, in_w, weight, rows, count, hidden, eps, out, stream);
    case 2: return launch_hyper_norm<T, 2>(x, y, mix_w, out_w, in_w, weight, rows, count, hidden, eps, out, stream);
    case 3: return launch_hyper_norm<T, 3>(x, y, mix_w, out_w, in_w, weight, rows, count, hidden, eps, out, stream);
    case 4: return launch_hyper_norm<T, 4>(x, y, mix_w, out_w, in_w, weight, rows, count, hidden, eps, out, stream);
    case 5: return launch_hyper_norm<T, 5>(x, y, mix_w, out_w, in_w, weight, rows, count, hidden, eps, out, stream);
    case 6: return launch_hyper_norm<T, 6>(x, y, mix_w, out_w, in_w, weight, rows, count, hidden, eps, out, stream);
    case 7: return launch_hyper_norm<T, 7>(x, y, mix_w, out_w, in_w, weight, rows, count, hidden, eps, out, stream);
    default: return launch_hyper_norm<T, 8>(x, y, mix_w, out_w, in_w, weight, rows, count, hidden, eps, out, stream);
  }
}

}  // namespace

B200_API int b200_embedding_sinusoid(const void* table, const int* ids, const int* positions, const float* inv_freq, float scale,
                                     float* out, int tokens, int streams, int hidden, int vocab, int dtype, int* err,
                                     cudaStream_t stream) {
  if (tokens == 0) return 0;
  B200_REQUIRE(tokens > 0 && hidden > 0 && hidden % 2 == 0 && vocab > 0 && streams > 0, "embedding_sinusoid: bad sizes");
  const int threads = hidden >= 2048 ? 256 : 128;
  if (dtype == DTYPE_F32) {
    launch_kernel(embedding_sinusoid_kernel<float>, dim3(tokens), dim3(threads), 0, stream, static_cast<const float*>(table), ids,
                  positions, inv_freq, scale, out, streams, hidden, vocab, err);
  } else if (dtype == DTYPE_BF16) {
    launch_kernel(embedding_sinusoid_kernel<__nv_bfloat16>, dim3(tokens), dim3(threads), 0, stream,
                  static_cast<const __nv_bfloat16*>(table), ids, positions, inv_freq, scale, out, streams, hidden, vocab, err);
  } else {
    return b200_fail("embedding_sinusoid: unknown dtype %d", dtype);
  }
  return b200_check_launch("embedding_sinusoid");
}

B200_API int b200_hyper_norm(float* x, const void* y, const float* mix_w, const float* out_w, const float* in_w, const float* weight,
                             const int* rows, int count, int streams, int hidden, float eps, void* out, int dtype,
                             cudaStream_t stream) {
  if (count == 0) return 0;
  B200_REQUIRE(count > 0 && hidden > 0 && streams > 0 && streams <= kMaxStreams, "hyper_norm: bad sizes (at most %d streams)", kMaxStreams);
  B200_REQUIRE(sizeof(float) * hidden <= 200 * 1024, "hyper_norm: a row of %d columns does not fit shared memory", hidden);
  B200_REQUIRE(y == nullptr || (mix_w != nullptr && out_w != nullptr), "hyper_norm: a branch output needs its mixing weights");
  if (dtype == DTYPE_F32) return dispatch_hyper_norm<float>(streams, x, y, mix_w, out_w, in_w, weight, rows, count, hidden, eps, out, stream);
  if (dtype == DTYPE_BF16)
    return dispatch_hyper_norm<__nv_bfloat16>(streams, x, y, mix_w, out_w, in_w, weight, rows, count, hidden, eps, out, stream);
  return b200_fail("hyper_norm: unknown dtype %d", dtype);
}

B200_API int b200_softcap(float* logits, int64_t count, float cap, cudaStream_t stream) {
  if (count == 0) return 0;
  B200_REQUIRE(count > 0 && cap > 0.f, "softcap: bad sizes");
  const int threads = 256;
  const int64_t blocks = (count + threads - 1) / threads;
  launch_kernel(softcap_kernel, dim3(static_cast<unsigned>(blocks < 4096 ? blocks : 4096)), dim3(threads), 0, stream, logits, count, cap);
  return b200_check_launch("softcap");
}
