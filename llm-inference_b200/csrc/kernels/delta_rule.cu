// The gated delta rule with one decay per head and key channel, and what surrounds it.
//
// Per head, with a state S [dk][dv] that starts at zero and is carried from token to token:
//   S <- g (.) S (g scales the rows of S, one factor per key channel);  u = beta (v - S^T k);
//   S <- S + k u^T;  o = S^T q   (the read-out sees the token's own write).
// q and k are unit vectors per head (q also times dk^-1/2) made from projections that first pass
// a short causal convolution over time and silu; g = exp(-exp(A_log[h]) softplus(a + dt_bias));
// beta = sigmoid(b). The state and the convolution's last taps - 1 inputs live in per-request
// slots. Everything that enters the recurrence is 32-bit.
//
// Kernels: `delta_prepare` (one block per token: convolution, silu, unit vectors, beta, decay),
// `conv_state_update` (one block per request: the slot's last inputs), `delta_recurrence` (the
// columns of S are independent, so a thread group owns a column and walks the request's tokens),
// `delta_output` (o / rms(o) * w * sigmoid(gate)).
#include "common.cuh"

namespace {

__device__ __forceinline__ float sigmoid_f(float x) { return 1.f / (1.f + expf(-x)); }
__device__ __forceinline__ float softplus_f(float x) { return x > 20.f ? x : log1pf(expf(x)); }

// `proj` rows: [q (kv_heads*dk) | k (kv_heads*dk) | v (heads*dv) | b (heads)]; the first
// `channels` = 2 kv_heads dk + heads dv columns pass the convolution. `conv_state`
// [slots][taps-1][channels] holds each request's last inputs, oldest first. `decay_in`
// [tokens][heads*dk] is W_a2 W_a1 h.
template <typename T>
__global__ void delta_prepare_kernel(const T* proj, int ld, const T* decay_in, int decay_ld,
                                     const float* __restrict__ taps_w, int taps, const T* conv_state,
                                     const float* __restrict__ a_log, const float* __restrict__ dt_bias,
                                     const int* token_seq, const int* seq_q_start, const int* seq_slot, int heads,
                                     int kv_heads, int dk, int dv, float* q_out, float* k_out, float* v_out, float* beta_out,
                                     float* decay_out) {
  extern __shared__ float y[];  // [channels]
  wait_for_predecessor();
  let_successor_start();
  const int t = blockIdx.x, tid = threadIdx.x;
  const int qk = kv_heads * dk, vw = heads * dv;
  const int channels = 2 * qk + vw;
  const int seq = token_seq[t];
  const int run = t - seq_q_start[seq];  // tokens of this request in front of t within the step
  const T* state = conv_state + static_cast<int64_t>(seq_slot[seq]) * (taps - 1) * channels;
  for (int c = tid; c < channels; c += blockDim.x) {
    float acc = 0.f;
    for (int j = 0; j < taps; ++j) {
      const int back = taps - 1 - j;  // how many tokens before t
      const float x = back <= run ? to_f32<T>(proj[static_cast<int64_t>(t - back) * ld + c])
                                  : to_f32<T>(state[static_cast<int64_t>(taps - 1 + run - back) * channels + c]);
      acc = fmaf(taps_w[c * taps + j], x, acc);
    }
    y[c] = acc * sigmoid_f(acc);
  }
  __syncthreads();
  const int lane = tid & 31, warp = tid >> 5, warps = blockDim.x >> 5;
  // unit vectors: one warp per (q or k, kv head)
  for (int item = warp; item < 2 * kv_heads; item += warps) {
    const float* src = y + item * dk;
    float ss = 0.f;
    for (int i = lane; i < dk; i += 32) ss = fmaf(src[i], src[i], ss);
    ss = warp_sum(ss);
    const bool is_q = item < kv_heads;
    const float factor = (1.f / sqrtf(ss + 1e-6f)) * (is_q ? 1.f / sqrtf(static_cast<float>(dk)) : 1.f);
    float* dst = (is_q ? q_out : k_out) + static_cast<int64_t>(t) * qk + (is_q ? item : item - kv_heads) * dk;
    for (int i = lane; i < dk; i += 32) dst[i] = src[i] * factor;
  }
  for (int i = tid; i < vw; i += blockDim.x) v_out[static_cast<int64_t>(t) * vw + i] = y[2 * qk + i];
  for (int h = tid; h < heads; h += blockDim.x)
    beta_out[static_cast<int64_t>(t) * heads + h] = sigmoid_f(to_f32<T>(proj[static_cast<int64_t>(t) * ld + channels + h]));
  for (int i = tid; i < heads * dk; i += blockDim.x) {
    const float step = softplus_f(to_f32<T>(decay_in[static_cast<int64_t>(t) * decay_ld + i]) + dt_bias[i]);
    decay_out[static_cast<int64_t>(t) * heads * dk + i] = expf(-expf(a_log[i / dk]) * step);
  }
}

// After a step the slot holds the last taps - 1 inputs of [old slot | the step's inputs].
template <typename T>
__global__ void conv_state_update_kernel(const T* proj, int ld, int channels, int taps, const int* seq_q_start,
                                         const int* seq_q_len, const int* seq_slot, T* conv_state) {
  wait_for_predecessor();
  let_successor_start();
  const int seq = blockIdx.x;
  const int start = seq_q_start[seq], len = seq_q_len[seq];
  const int keep = taps - 1;
  T* state = conv_state + static_cast<int64_t>(seq_slot[seq]) * keep * channels;
  for (int c = threadIdx.x; c < channels; c += blockDim.x) {
    for (int r = 0; r < keep; ++r) {
      const int at = len + r;  // index into [old slot (keep) | inputs (len)]
      state[static_cast<int64_t>(r) * channels + c] =
          at < keep ? state[static_cast<int64_t>(at) * channels + c] : proj[static_cast<int64_t>(start + at - keep) * ld + c];
    }
  }
}

// A block owns `cols` columns of one head of one request; a column's dk rows are spread over
// `lanes_per_col` neighbouring lanes (row r on lane r % lanes_per_col), PER rows per lane in
// registers: few rows per lane keep the two dot products' chains of dependent FMAs short, which
// is what a token's latency is made of. The tokens' q, k, g, v and beta arrive kStage at a time
// by cp.async in a ring of two stages, so the next tokens load while these are worked on.
constexpr int kRecurrenceThreads = 128;
constexpr int kStage = 8;

// `bytes` (4 or 16) global -> shared; with `valid` false zeros are written and nothing is read.
template <int kBytes>
__device__ __forceinline__ void stage_copy(float* smem, const float* gmem, bool valid) {
  const uint32_t s = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
  const int bytes = valid ? kBytes : 0;
  asm volatile("cp.async.ca.shared.global [%0], [%1], %2, %3;" ::"r"(s), "l"(gmem), "n"(kBytes), "r"(bytes) : "memory");
}

template <int PER, int LANES>
__global__ void __launch_bounds__(kRecurrenceThreads)
delta_recurrence_kernel(const float* q, const float* k, const float* v, const float* beta, const float* decay,
                        const int* seq_q_start, const int* seq_q_len, const int* seq_slot, int heads, int kv_heads, int dk,
                        int dv, int vec, float* state, float* out) {
  extern __shared__ __align__(16) float stage[];
  let_successor_start();
  constexpr int lanes_per_col = LANES;
  constexpr int cols = kRecurrenceThreads / lanes_per_col;
  const int seq = blockIdx.x, head = blockIdx.y, col0 = blockIdx.z * cols;
  const int tid = threadIdx.x;
  const int part = tid % lanes_per_col, col = col0 + tid / lanes_per_col;
  constexpr int padded = PER * lanes_per_col;
  constexpr int per_stage = kStage * (3 * padded + cols) + kStage;
  const int start = seq_q_start[seq], len = seq_q_len[seq];
  const int kvh = head / (heads / kv_heads);
  const bool live = col < dv;
  float* s_base = state + (static_cast<int64_t>(seq_slot[seq]) * heads + head) * dk * dv;
  wait_for_predecessor();
  // Rows past dk (when dk is no multiple of the lanes) hold zeros in q, k and g and stay zero.
  auto fetch = [&](int buffer, int t0) {
    float* sq = stage + buffer * per_stage;
    float* sk = sq + kStage * padded;
    float* sg = sk + kStage * padded;
    float* sv = sg + kStage * padded;
    float* sb = sv + kStage * cols;
    const int count = min(kStage, len - t0);
    const int64_t first = static_cast<int64_t>(start) + t0;
    if (vec) {
      for (int idx = tid * 4; idx < count * padded; idx += kRecurrenceThreads * 4) {
        const int j = idx / padded, r = idx % padded;
        const int64_t tok = first + j;
        const bool in = r < dk;
        const int rr = in ? r : 0;
        stage_copy<16>(sq + idx, q + (tok * kv_heads + kvh) * dk + rr, in);
        stage_copy<16>(sk + idx, k + (tok * kv_heads + kvh) * dk + rr, in);
        stage_copy<16>(sg + idx, decay + (tok * heads + head) * dk + rr, in);
      }
      for (int idx = tid * 4; idx < count * cols; idx += kRecurrenceThreads * 4) {
        const int j = idx / cols, c = col0 + idx % cols;
        stage_copy<16>(sv + idx, v + ((first + j) * heads + head) * dv + (c < dv ? c : 0), c < dv);
      }
    } else {
      for (int idx = tid; idx < count * padded; idx += kRecurrenceThreads) {
        const int j = idx / padded, r = idx % padded;
        const int64_t tok = first + j;
        const bool in = r < dk;
        const int rr = in ? r : 0;
        stage_copy<4>(sq + idx, q + (tok * kv_heads + kvh) * dk + rr, in);
        stage_copy<4>(sk + idx, k + (tok * kv_heads + kvh) * dk + rr, in);
        stage_copy<4>(sg + idx, decay + (tok * heads + head) * dk + rr, in);
      }
      for (int idx = tid; idx < count * cols; idx += kRecurrenceThreads) {
        const int j = idx / cols, c = col0 + idx % cols;
        stage_copy<4>(sv + idx, v + ((first + j) * heads + head) * dv + (c < dv ? c : 0), c < dv);
      }
    }
    if (tid < count) stage_copy<4>(sb + tid, beta + (first + tid) * heads + head, true);
  };
  float s[PER];
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    const int r = i * lanes_per_col + part;
    s[i] = (live && r < dk) ? s_base[static_cast<int64_t>(r) * dv + col] : 0.f;
  }
  if (len > 0) fetch(0, 0);
  asm volatile("cp.async.commit_group;" ::: "memory");
  for (int t0 = 0, buffer = 0; t0 < len; t0 += kStage, buffer ^= 1) {
    if (t0 + kStage < len) fetch(buffer ^ 1, t0 + kStage);
    asm volatile("cp.async.commit_group;" ::: "memory");
    asm volatile("cp.async.wait_group 1;" ::: "memory");
    __syncthreads();
    const float* sq = stage + buffer * per_stage;
    const float* sk = sq + kStage * padded;
    const float* sg = sk + kStage * padded;
    const float* sv = sg + kStage * padded;
    const float* sb = sv + kStage * cols;
    const int count = min(kStage, len - t0);
    for (int j = 0; j < count; ++j) {
      const float* kj = sk + j * padded + part;
      const float* gj = sg + j * padded + part;
      const float* qj = sq + j * padded + part;
      float kr[PER];
      float ks0 = 0.f, ks1 = 0.f;
#pragma unroll
      for (int i = 0; i < PER; i += 2) {
        kr[i] = kj[i * lanes_per_col], kr[i + 1] = kj[(i + 1) * lanes_per_col];
        s[i] *= gj[i * lanes_per_col], s[i + 1] *= gj[(i + 1) * lanes_per_col];
        ks0 = fmaf(kr[i], s[i], ks0), ks1 = fmaf(kr[i + 1], s[i + 1], ks1);
      }
      float ks = ks0 + ks1;
#pragma unroll
      for (int o = lanes_per_col >> 1; o > 0; o >>= 1) ks += __shfl_xor_sync(0xffffffffu, ks, o);
      const float u = sb[j] * (sv[j * cols + tid / lanes_per_col] - ks);
      float qs0 = 0.f, qs1 = 0.f;
#pragma unroll
      for (int i = 0; i < PER; i += 2) {
        s[i] = fmaf(kr[i], u, s[i]), s[i + 1] = fmaf(kr[i + 1], u, s[i + 1]);
        qs0 = fmaf(qj[i * lanes_per_col], s[i], qs0), qs1 = fmaf(qj[(i + 1) * lanes_per_col], s[i + 1], qs1);
      }
      float qs = qs0 + qs1;
#pragma unroll
      for (int o = lanes_per_col >> 1; o > 0; o >>= 1) qs += __shfl_xor_sync(0xffffffffu, qs, o);
      if (live && part == 0) out[(static_cast<int64_t>(start) + t0 + j) * heads * dv + head * dv + col] = qs;
    }
    __syncthreads();
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    const int r = i * lanes_per_col + part;
    if (live && r < dk) s_base[static_cast<int64_t>(r) * dv + col] = s[i];
  }
}

// out[t, h, :] = o / rms(o) * w * sigmoid(gate[t, h, :]); one warp per (token, head).
template <typename T>
__global__ void delta_output_kernel(const float* o, const float* __restrict__ weight, const T* gate, int gate_ld, int rows,
                                    int heads, int dv, float eps, T* out) {
  wait_for_predecessor();
  let_successor_start();
  const int lane = threadIdx.x & 31;
  const int item = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (item >= rows * heads) return;
  const int t = item / heads, h = item % heads;
  const float* src = o + static_cast<int64_t>(item) * dv;
  float ss = 0.f;
  for (int i = lane; i < dv; i += 32) ss = fmaf(src[i], src[i], ss);
  ss = warp_sum(ss);
  const float inv = 1.f / sqrtf(ss / static_cast<float>(dv) + eps);
  const T* g = gate + static_cast<int64_t>(t) * gate_ld + h * dv;
  T* dst = out + static_cast<int64_t>(item) * dv;
  for (int i = lane; i < dv; i += 32) dst[i] = from_f32<T>(src[i] * inv * weight[i] * sigmoid_f(to_f32<T>(g[i])));
}

}  // namespace

B200_API int b200_delta_prepare(const void* proj, int ld, const void* decay_in, int decay_ld, const float* taps_w, int taps,
                                void* conv_state, const float* a_log, const float* dt_bias, const int* token_seq,
                                const int* seq_q_start, const int* seq_q_len, const int* seq_slot, int tokens, int seqs,
                                int heads, int kv_heads, int dk, int dv, float* q_out, float* k_out, float* v_out,
                                float* beta_out, float* decay_out, int dtype, cudaStream_t stream) {
  if (tokens == 0) return 0;
  B200_REQUIRE(tokens > 0 && seqs > 0 && heads > 0 && kv_heads > 0 && heads % kv_heads == 0 && dk > 0 && dv > 0 && taps >= 1,
               "delta_prepare: bad sizes");
  const int channels = 2 * kv_heads * dk + heads * dv;
  const size_t smem = sizeof(float) * channels;
  B200_REQUIRE(smem <= 200 * 1024, "delta_prepare: %d convolved channels do not fit shared memory", channels);
  const int threads = 256;
  if (dtype == DTYPE_F32) {
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(delta_prepare_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    launch_kernel(delta_prepare_kernel<float>, dim3(tokens), dim3(threads), smem, stream, static_cast<const float*>(proj), ld,
                  static_cast<const float*>(decay_in), decay_ld, taps_w, taps, static_cast<const float*>(conv_state), a_log,
                  dt_bias, token_seq, seq_q_start, seq_slot, heads, kv_heads, dk, dv, q_out, k_out, v_out, beta_out, decay_out);
    if (int status = b200_check_launch("delta_prepare")) return status;
    launch_kernel(conv_state_update_kernel<float>, dim3(seqs), dim3(threads), 0, stream, static_cast<const float*>(proj), ld,
                  channels, taps, seq_q_start, seq_q_len, seq_slot, static_cast<float*>(conv_state));
  } else if (dtype == DTYPE_BF16) {
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(delta_prepare_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           static_cast<int>(smem));
    launch_kernel(delta_prepare_kernel<__nv_bfloat16>, dim3(tokens), dim3(threads), smem, stream,
                  static_cast<const __nv_bfloat16*>(proj), ld, static_cast<const __nv_bfloat16*>(decay_in), decay_ld, taps_w,
                  taps, static_cast<const __nv_bfloat16*>(conv_state), a_log, dt_bias, token_seq, seq_q_start, seq_slot, heads,
                  kv_heads, dk, dv, q_out, k_out, v_out, beta_out, decay_out);
    if (int status = b200_check_launch("delta_prepare")) return status;
    launch_kernel(conv_state_update_kernel<__nv_bfloat16>, dim3(seqs), dim3(threads), 0, stream,
                  static_cast<const __nv_bfloat16*>(proj), ld, channels, taps, seq_q_start, seq_q_len, seq_slot,
                  static_cast<__nv_bfloat16*>(conv_state));
  } else {
    return b200_fail("delta_prepare: unknown dtype %d", dtype);
  }
  return b200_check_launch("conv_state_update");
}

B200_API int b200_delta_recurrence(const float* q, const float* k, const float* v, const float* beta, const float* decay,
                                   const int* seq_q_start, const int* seq_q_len, const int* seq_slot, int seqs, int heads,
                                   int kv_heads, int dk, int dv, float* state, float* out, cudaStream_t stream) {
  if (seqs == 0) return 0;
  B200_REQUIRE(seqs > 0 && heads > 0 && heads <= 65535 && kv_heads > 0 && heads % kv_heads == 0 && dk > 0 && dv > 0,
               "delta_recurrence: bad sizes");
  B200_REQUIRE(dk <= 1024, "delta_recurrence: %d key channels per head, at most 1024", dk);
  // Lanes per column: enough that a lane holds at most 8 rows (up to 32 rows when even a whole warp
  // per column leaves more).
  int lanes = 1;
  while ((dk + lanes - 1) / lanes > 8 && lanes < 32) lanes *= 2;
  const int rows = (dk + lanes - 1) / lanes;
  B200_REQUIRE(rows <= 32, "delta_recurrence: %d key channels per head, at most 1024", dk);
  const int per = rows <= 8 ? 8 : (rows <= 16 ? 16 : 32);
  const int cols = kRecurrenceThreads / lanes;
  const dim3 grid(seqs, heads, (dv + cols - 1) / cols);
  B200_REQUIRE(grid.z <= 65535, "delta_recurrence: too many columns");
  const size_t smem = sizeof(float) * 2 * (kStage * (3 * per * lanes + cols) + kStage);
  const auto aligned = [](const void* p) { return reinterpret_cast<uintptr_t>(p) % 16 == 0; };
  // 16-byte copies when every staged row starts on a 16-byte boundary.
  const int vec = dk % 4 == 0 && dv % 4 == 0 && aligned(q) && aligned(k) && aligned(v) && aligned(decay) ? 1 : 0;
  B200_REQUIRE(smem <= 200 * 1024, "delta_recurrence: the staged tokens do not fit shared memory");
  auto launch = [&](auto kernel) {
    if (smem > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    launch_kernel(kernel, grid, dim3(kRecurrenceThreads), smem, stream, q, k, v, beta, decay, seq_q_start, seq_q_len, seq_slot,
                  heads, kv_heads, dk, dv, vec, state, out);
  };
  if (per == 32) launch(delta_recurrence_kernel<32, 32>);
  else if (per == 16) launch(delta_recurrence_kernel<16, 32>);
  else if (lanes == 32) launch(delta_recurrence_kernel<8, 32>);
  else if (lanes == 16) launch(delta_recurrence_kernel<8, 16>);
  else if (lanes == 8) launch(delta_recurrence_kernel<8, 8>);
  else if (lanes == 4) launch(delta_recurrence_kernel<8, 4>);
  else if (lanes == 2) launch(delta_recurrence_kernel<8, 2>);
  else launch(delta_recurrence_kernel<8, 1>);
  return b200_check_launch("delta_recurrence");
}

B200_API int b200_delta_output(const float* o, const float* weight, const void* gate, int gate_ld, int rows, int heads, int dv,
                               float eps, void* out, int dtype, cudaStream_t stream) {
  if (rows == 0) return 0;
  B200_REQUIRE(rows > 0 && heads > 0 && dv > 0, "delta_output: bad sizes");
  const int threads = 128;
  const int64_t items = static_cast<int64_t>(rows) * heads;
  const unsigned blocks = static_cast<unsigned>((items + 3) / 4);
  if (dtype == DTYPE_F32) {
    launch_kernel(delta_output_kernel<float>, dim3(blocks), dim3(threads), 0, stream, o, weight, static_cast<const float*>(gate),
                  gate_ld, rows, heads, dv, eps, static_cast<float*>(out));
  } else if (dtype == DTYPE_BF16) {
    launch_kernel(delta_output_kernel<__nv_bfloat16>, dim3(blocks), dim3(threads), 0, stream, o, weight,
                  static_cast<const __nv_bfloat16*>(gate), gate_ld, rows, heads, dv, eps, static_cast<__nv_bfloat16*>(out));
  } else {
    return b200_fail("delta_output: unknown dtype %d", dtype);
  }
  return b200_check_launch("delta_output");
}
