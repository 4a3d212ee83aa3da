// Attention over cached latents on tensor cores (bfloat16), for prompt portions and for single tokens.
//
// All heads of a request read the same cached rows [latent (rank) | rotated key part (rot_dim)],
// and a head's value is the latent itself (see latent_attention.cu), so the (token, head) pairs
// of a request's new tokens are the rows of one matrix problem: S = Q K^T over rows of
// rank + rot_dim numbers, O = P K[:, :rank]. A block owns 16 * RW consecutive rows (row r is token
// r / heads, head r % heads) and walks the keys 32 at a time: a tile's rows arrive as bulk copies
// (`cp.async.bulk`, one per key, issued by the lanes of warp 0 and counted on an mbarrier per
// stage) straight from the pages into a ring of two stages, so the warps that compute spend no
// issue slots on loads; scores and P V run on `mma.sync` m16n8k16 with 32-bit
// accumulators, the softmax is the usual running maximum and sum in 32-bit (base 2, the scale
// folded in), started at (sink, 1): the sink's term. Two warps share 16 rows: each forms the scores
// over one half of the row's numbers, they swap their partial sums through shared memory (one
// named barrier of 64 threads per tile) so that both hold the same scores and weights, and each
// keeps one half of the value columns in registers (rank / 4 of them per thread).
// Rows of keys past a request's end are never read from a page: their place in shared memory holds
// zeros or an earlier tile's rows, and their weights are zero. Every wait on an mbarrier gives up
// after about two seconds, sets a bit in the error word and ends the block.
// With gridDim.z > 1 the keys are cut into that many pieces whose (maximum, sum, unnormalised
// output) go to scratch and a second kernel merges them: single tokens have too few rows to fill
// the GPU otherwise. The output gate sigmoid(gate[t, h]) is applied on the way out.
#include "common.cuh"

namespace {

constexpr int kKeys = 32;  // keys per tile
constexpr int kPad = 8;    // bfloat16 elements between shared-memory rows: neighbouring rows start 4 banks apart
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLowest = -1e30f;  // a finite "no maximum yet": differences of two of them stay finite

struct LatentParams {
  const __nv_bfloat16* q_lat;  // [token][head][rank] through the two strides
  int64_t q_lat_token, q_lat_head;
  const __nv_bfloat16* q_rot;  // [token][head][rot_dim]
  const __nv_bfloat16* arena;  // [page][row][rank + rot_dim]
  const int* block_table;
  int max_pages, num_pages, page_size;
  const int* seq_q_start;
  const int* seq_q_len;
  const int* seq_kv_len;
  int first_seq;
  const float* sink;            // [heads] or null
  const __nv_bfloat16* gate;    // [token][gate_ld] logits or null
  int64_t gate_ld;
  __nv_bfloat16* out;           // [token][head][rank] through the two strides
  int64_t out_token, out_head;
  float* partial;               // [seq][row][piece][2 + rank] when the keys are cut
  int rows_cap;                 // rows per request in `partial`
  int heads, rank, rot_dim;
  float scale_log2;
  int stages;                   // K tiles in flight: 3 where shared memory allows, else 2
  int* err;
};

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* p) {
  const uint32_t a = static_cast<uint32_t>(__cvta_generic_to_shared(p));
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* p) {
  const uint32_t a = static_cast<uint32_t>(__cvta_generic_to_shared(p));
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// 16 bytes global -> shared; with `valid` false nothing is read and zeros are written.
__device__ __forceinline__ void copy16(void* smem, const void* gmem, bool valid) {
  const uint32_t s = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
  const int bytes = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(s), "l"(gmem), "r"(bytes) : "memory");
}
constexpr long long kWaitCycles = 4000000000LL;  // about two seconds
constexpr int ERRBIT_TIMEOUT_L = 8;                // "a kernel gave up waiting on one of its own barriers"

__device__ __forceinline__ uint32_t shared_address(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ void ring_init(uint64_t* bar) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(shared_address(bar)) : "memory");
}
__device__ __forceinline__ void ring_expect(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(shared_address(bar)), "r"(bytes) : "memory");
}
// `bytes` (a multiple of 16, both addresses 16-byte aligned) global -> shared, counted on `bar`.
__device__ __forceinline__ void bulk_copy(void* smem, const void* gmem, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(shared_address(smem)), "l"(gmem), "r"(bytes), "r"(shared_address(bar)) : "memory");
}
__device__ __forceinline__ bool ring_wait(uint64_t* bar, uint32_t parity) {
  const uint32_t addr = shared_address(bar);
  const long long start = clock64();
  while (true) {
    uint32_t done;
    asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}\n"
                 : "=r"(done) : "r"(addr), "r"(parity) : "memory");
    if (done) return true;
    if (clock64() - start > kWaitCycles) return false;
  }
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
}

// A barrier of the two warps that share 16 rows (named barrier 1 + pair; 0 is the block's). The
// number is an immediate so that the block is charged for the barriers it uses, not for all 16.
__device__ __forceinline__ void pair_barrier(int pair) {
  switch (pair) {
    case 0: asm volatile("bar.sync 1, 64;" ::: "memory"); break;
    case 1: asm volatile("bar.sync 2, 64;" ::: "memory"); break;
    case 2: asm volatile("bar.sync 3, 64;" ::: "memory"); break;
    default: asm volatile("bar.sync 4, 64;" ::: "memory"); break;
  }
}

template <int RW, int VH_MAX>
__global__ void __launch_bounds__(64 * RW, 1) latent_attention_mma_kernel(const LatentParams p) {
  constexpr int BM = 16 * RW, kThreads = 64 * RW;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int width = p.rank + p.rot_dim, ld = width + kPad, chunks = width / 8;
  __nv_bfloat16* qs = reinterpret_cast<__nv_bfloat16*>(smem_raw);  // [BM][ld]
  __nv_bfloat16* ks = qs + BM * ld;                                // [stages][kKeys][ld]
  float* swap = reinterpret_cast<float*>(ks + p.stages * kKeys * ld);  // [2][RW][2][16][32] partial scores
  let_successor_start();
  const int seq = p.first_seq + blockIdx.y;
  const int q_start = p.seq_q_start[seq], q_len = p.seq_q_len[seq], kv_len = p.seq_kv_len[seq];
  wait_for_predecessor();
  const int rows_total = q_len * p.heads;
  const int blocks = (rows_total + BM - 1) / BM;
  if (static_cast<int>(blockIdx.x) >= blocks) return;
  const int block = blocks - 1 - blockIdx.x;  // the rows with the most keys first
  const int row0 = block * BM;
  const int first_pos = kv_len - q_len;
  const int max_pos = first_pos + (min(row0 + BM, rows_total) - 1) / p.heads;
  const int tiles = max_pos / kKeys + 1;
  const int pieces = gridDim.z, piece = blockIdx.z;
  const int per = (tiles + pieces - 1) / pieces;
  const int tile_begin = piece * per, tile_end = min(tiles, tile_begin + per);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int rw = warp >> 1, half = warp & 1;
  const int vh = p.rank / 2;
  const int* table = p.block_table + static_cast<int64_t>(seq) * p.max_pages;

  // queries of this block's rows
  for (int idx = tid; idx < BM * chunks; idx += kThreads) {
    const int r = idx / chunks, col = (idx % chunks) * 8;
    const int g = row0 + r;
    const bool valid = g < rows_total;
    const int token = q_start + (valid ? g / p.heads : 0), head = valid ? g % p.heads : 0;
    const __nv_bfloat16* src = col < p.rank ? p.q_lat + token * p.q_lat_token + head * p.q_lat_head + col
                                            : p.q_rot + (static_cast<int64_t>(token) * p.heads + head) * p.rot_dim + (col - p.rank);
    copy16(qs + r * ld + col, src, valid);
  }
  // The ring's barriers; its stages start as zeros (a tile's rows past the request's end are never copied).
  __shared__ __align__(8) uint64_t full[3];
  if (tid == 0) {
    for (int i = 0; i < p.stages; ++i) ring_init(&full[i]);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  for (int i = tid; i < p.stages * kKeys * ld / 8; i += kThreads) reinterpret_cast<uint4*>(ks)[i] = make_uint4(0u, 0u, 0u, 0u);
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  __syncthreads();
  // A tile is 32 keys: lane i of warp 0 looks up the page of key i and asks for that row as one bulk copy.
  auto load_tile = [&](int stage, int tile) {
    if (warp != 0) return;
    __nv_bfloat16* dst = ks + stage * kKeys * ld;
    const int mine = tile * kKeys + lane;
    int64_t my_row = -1;
    if (mine <= max_pos) {
      const int logical = mine / p.page_size;
      const int page = logical < p.max_pages ? table[logical] : -1;
      if (page < 0 || page >= p.num_pages) atomicOr(p.err, ERRBIT_BAD_PAGE);
      else my_row = static_cast<int64_t>(page) * p.page_size + mine % p.page_size;
    }
    const uint32_t row_bytes = static_cast<uint32_t>(width) * 2u;
    const int rows = __popc(__ballot_sync(0xffffffffu, my_row >= 0));
    if (lane == 0) ring_expect(&full[stage], rows * row_bytes);
    __syncwarp();
    if (my_row >= 0) bulk_copy(dst + lane * ld, p.arena + my_row * width, row_bytes, &full[stage]);
  };

  // this thread's two rows: lane / 4 and lane / 4 + 8 of the warp pair's sixteen
  const int r_lo = row0 + rw * 16 + (lane >> 2), r_hi = r_lo + 8;
  const int pos_lo = r_lo < rows_total ? first_pos + r_lo / p.heads : -1;
  const int pos_hi = r_hi < rows_total ? first_pos + r_hi / p.heads : -1;
  const int pair_first = row0 + rw * 16;
  const int pair_max_pos = pair_first < rows_total ? first_pos + (min(pair_first + 16, rows_total) - 1) / p.heads : -1;
  float m_lo = kLowest, m_hi = kLowest, l_lo = 0.f, l_hi = 0.f;
  if (p.sink && piece == 0) {
    if (pos_lo >= 0) m_lo = p.sink[r_lo % p.heads] * kLog2e, l_lo = (lane & 3) == 0 ? 1.f : 0.f;
    if (pos_hi >= 0) m_hi = p.sink[r_hi % p.heads] * kLog2e, l_hi = (lane & 3) == 0 ? 1.f : 0.f;
  }
  float o[VH_MAX / 8][4];
#pragma unroll
  for (int i = 0; i < VH_MAX / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;

  // The ring: tiles i + 1 .. i + stages - 1 are on their way while tile i is worked on. The one
  // block barrier per tile says both that tile i has landed for everybody and that everybody has
  // left tile i - 1, whose stage the next copies overwrite.
  const int stages = p.stages;
  int asked = 0;  // tiles whose copies were issued (same count in every thread)
  for (; asked < stages - 1 && tile_begin + asked < tile_end; ++asked) load_tile(asked, tile_begin + asked);
  asm volatile("cp.async.commit_group;" ::: "memory");
  asm volatile("cp.async.wait_group 0;" ::: "memory");  // the queries
  bool gave_up = false;
  for (int tile = tile_begin; tile < tile_end; ++tile) {
    const int turn = tile - tile_begin;
    const int stage = turn % stages;
    const bool landed = ring_wait(&full[stage], (turn / stages) & 1);
    if (__syncthreads_or(!landed)) {
      gave_up = true;
      if (tid == 0) atomicOr(p.err, ERRBIT_TIMEOUT_L);
      // the copies still on their way get the same bounded time, then the block leaves
      for (int rest = turn + 1; rest < asked; ++rest) ring_wait(&full[rest % stages], (rest / stages) & 1);
      break;
    }
    if (tile_begin + asked < tile_end) {
      load_tile(asked % stages, tile_begin + asked);
      ++asked;
    }
    const int n0 = tile * kKeys;
    if (n0 <= pair_max_pos) {
      const __nv_bfloat16* kt = ks + stage * kKeys * ld;
      float s[4][4];
#pragma unroll
      for (int i = 0; i < 4; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
      const __nv_bfloat16* a_at = qs + (rw * 16 + (lane & 15)) * ld + (lane >> 4) * 8;
      const __nv_bfloat16* b_at = kt + ((lane & 7) + (lane >> 4) * 8) * ld + ((lane >> 3) & 1) * 8;
      const int k_cut = (width / 16 + 1) / 2 * 16;  // this warp's share of the row: [0, k_cut) or [k_cut, width)
#pragma unroll 2
      for (int k0 = half ? k_cut : 0; k0 < (half ? width : k_cut); k0 += 16) {
        uint32_t a[4], b[4];
        ldmatrix_x4(a, a_at + k0);
        ldmatrix_x4(b, b_at + k0);
        mma_bf16(s[0], a, b[0], b[1]);
        mma_bf16(s[1], a, b[2], b[3]);
        ldmatrix_x4(b, b_at + 16 * ld + k0);
        mma_bf16(s[2], a, b[0], b[1]);
        mma_bf16(s[3], a, b[2], b[3]);
      }
      {  // the pair's two partial sums meet: both warps add the same two numbers, so both hold the same scores
        float* mine = swap + (((turn & 1) * RW + rw) * 2 + half) * 512 + lane;
        const float* theirs = swap + (((turn & 1) * RW + rw) * 2 + (half ^ 1)) * 512 + lane;
#pragma unroll
        for (int i = 0; i < 16; ++i) mine[i * 32] = s[i >> 2][i & 3];
        pair_barrier(rw);
#pragma unroll
        for (int i = 0; i < 16; ++i) s[i >> 2][i & 3] += theirs[i * 32];
      }
      float top_lo = kLowest, top_hi = kLowest;
#pragma unroll
      for (int nt = 0; nt < 4; ++nt) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int key = n0 + nt * 8 + (lane & 3) * 2 + (e & 1);
          const bool seen = key <= (e < 2 ? pos_lo : pos_hi);
          s[nt][e] = seen ? s[nt][e] * p.scale_log2 : -INFINITY;
        }
        top_lo = fmaxf(top_lo, fmaxf(s[nt][0], s[nt][1]));
        top_hi = fmaxf(top_hi, fmaxf(s[nt][2], s[nt][3]));
      }
      top_lo = fmaxf(top_lo, __shfl_xor_sync(0xffffffffu, top_lo, 1));
      top_lo = fmaxf(top_lo, __shfl_xor_sync(0xffffffffu, top_lo, 2));
      top_hi = fmaxf(top_hi, __shfl_xor_sync(0xffffffffu, top_hi, 1));
      top_hi = fmaxf(top_hi, __shfl_xor_sync(0xffffffffu, top_hi, 2));
      const float new_lo = fmaxf(m_lo, top_lo), new_hi = fmaxf(m_hi, top_hi);
      const float alpha_lo = exp2f(m_lo - new_lo), alpha_hi = exp2f(m_hi - new_hi);
      m_lo = new_lo, m_hi = new_hi;
      float sum_lo = 0.f, sum_hi = 0.f;
#pragma unroll
      for (int nt = 0; nt < 4; ++nt) {
        s[nt][0] = exp2f(s[nt][0] - new_lo), s[nt][1] = exp2f(s[nt][1] - new_lo);
        s[nt][2] = exp2f(s[nt][2] - new_hi), s[nt][3] = exp2f(s[nt][3] - new_hi);
        sum_lo += s[nt][0] + s[nt][1];
        sum_hi += s[nt][2] + s[nt][3];
      }
      l_lo = l_lo * alpha_lo + sum_lo, l_hi = l_hi * alpha_hi + sum_hi;
#pragma unroll
      for (int i = 0; i < VH_MAX / 8; ++i) o[i][0] *= alpha_lo, o[i][1] *= alpha_lo, o[i][2] *= alpha_hi, o[i][3] *= alpha_hi;
      uint32_t pa[2][4];
#pragma unroll
      for (int kk = 0; kk < 2; ++kk) {
        pa[kk][0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
        pa[kk][1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
        pa[kk][2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
        pa[kk][3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
      }
      const __nv_bfloat16* v_at = kt + ((lane & 7) + ((lane >> 3) & 1) * 8) * ld + half * vh + (lane >> 4) * 8;
#pragma unroll
      for (int nv = 0; nv < VH_MAX / 16; ++nv) {
        if (nv * 16 < vh) {
#pragma unroll
          for (int kk = 0; kk < 2; ++kk) {
            uint32_t b[4];
            ldmatrix_x4_trans(b, v_at + kk * 16 * ld + nv * 16);
            mma_bf16(o[2 * nv], pa[kk], b[0], b[1]);
            mma_bf16(o[2 * nv + 1], pa[kk], b[2], b[3]);
          }
        }
      }
    }
  }
  if (gave_up) return;
  l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 1);
  l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 2);
  l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 1);
  l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 2);
#pragma unroll
  for (int side = 0; side < 2; ++side) {
    const int g = side ? r_hi : r_lo;
    if (g >= rows_total) continue;
    const int token = q_start + g / p.heads, head = g % p.heads;
    const float m = side ? m_hi : m_lo, l = side ? l_hi : l_lo;
    if (pieces == 1) {
      float factor = l > 0.f ? 1.f / l : 0.f;
      if (p.gate) factor *= 1.f / (1.f + expf(-__bfloat162float(p.gate[token * p.gate_ld + head])));
      __nv_bfloat16* dst = p.out + token * p.out_token + head * p.out_head + half * vh + (lane & 3) * 2;
#pragma unroll
      for (int i = 0; i < VH_MAX / 8; ++i)
        if (i * 8 < vh)
          *reinterpret_cast<__nv_bfloat162*>(dst + i * 8) = __floats2bfloat162_rn(o[i][2 * side] * factor, o[i][2 * side + 1] * factor);
    } else {
      float* dst = p.partial + ((static_cast<int64_t>(blockIdx.y) * p.rows_cap + g) * pieces + piece) * (p.rank + 2);
      if (half == 0 && (lane & 3) == 0) dst[0] = m, dst[1] = l;
      dst += 2 + half * vh + (lane & 3) * 2;
#pragma unroll
      for (int i = 0; i < VH_MAX / 8; ++i)
        if (i * 8 < vh) *reinterpret_cast<float2*>(dst + i * 8) = make_float2(o[i][2 * side], o[i][2 * side + 1]);
    }
  }
}

// One block per (row, request): the pieces' results weighed by 2^(m_piece - max), then the gate.
__global__ void latent_attention_merge_kernel(const float* partial, int pieces, int rows_cap, int rank, int heads, int first_seq,
                                              const int* seq_q_start, const int* seq_q_len, const __nv_bfloat16* gate,
                                              int64_t gate_ld, __nv_bfloat16* out, int64_t out_token, int64_t out_head) {
  let_successor_start();
  const int seq = first_seq + blockIdx.y, g = blockIdx.x;
  const int q_start = seq_q_start[seq], rows_total = seq_q_len[seq] * heads;
  wait_for_predecessor();
  if (g >= rows_total) return;
  const float* base = partial + (static_cast<int64_t>(blockIdx.y) * rows_cap + g) * pieces * (rank + 2);
  float top = kLowest;
  for (int s = 0; s < pieces; ++s) top = fmaxf(top, base[s * (rank + 2)]);
  float total = 0.f;
  for (int s = 0; s < pieces; ++s) total += exp2f(base[s * (rank + 2)] - top) * base[s * (rank + 2) + 1];
  const int token = q_start + g / heads, head = g % heads;
  float factor = total > 0.f ? 1.f / total : 0.f;
  if (gate) factor *= 1.f / (1.f + expf(-__bfloat162float(gate[token * gate_ld + head])));
  __nv_bfloat16* dst = out + token * out_token + head * out_head;
  for (int c = threadIdx.x; c < rank; c += blockDim.x) {
    float acc = 0.f;
    for (int s = 0; s < pieces; ++s) acc = fmaf(exp2f(base[s * (rank + 2)] - top), base[s * (rank + 2) + 2 + c], acc);
    dst[c] = __float2bfloat16_rn(acc * factor);
  }
}

constexpr size_t kSharedLimit = 225 * 1024;

size_t shared_bytes(int rw, int rank, int rot_dim, int stages) {
  return sizeof(__nv_bfloat16) * static_cast<size_t>(16 * rw + stages * kKeys) * (rank + rot_dim + kPad) + sizeof(float) * 2 * rw * 2 * 512;
}

template <int RW, int VH_MAX>
int launch(const LatentParams& p, dim3 grid, size_t smem, cudaStream_t stream) {
  static bool raised = false;  // per instantiation
  if (!raised) {
    if (cudaFuncSetAttribute(latent_attention_mma_kernel<RW, VH_MAX>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(kSharedLimit)) !=
        cudaSuccess)
      return b200_fail("latent_attention_mma: cannot raise the shared-memory limit");
    raised = true;
  }
  launch_kernel(latent_attention_mma_kernel<RW, VH_MAX>, grid, dim3(64 * RW), smem, stream, p);
  return b200_check_launch("latent_attention_mma");
}

template <int RW>
int launch_for_rank(const LatentParams& p, dim3 grid, size_t smem, cudaStream_t stream) {
  if (p.rank <= 128) return launch<RW, 64>(p, grid, smem, stream);
  if (p.rank <= 256) return launch<RW, 128>(p, grid, smem, stream);
  return launch<RW, 256>(p, grid, smem, stream);
}

}  // namespace

// Shapes the tensor-core kernel takes: a latent of a multiple of 32 up to 512 numbers, a rotated part
// of a multiple of 16, rows that fit shared memory beside 64 queries.
B200_API int b200_latent_attention_mma_supported(int heads, int rank, int rot_dim, int page_size) {
  return heads > 0 && rank > 0 && rank % 32 == 0 && rank <= 512 && rot_dim >= 0 && rot_dim % 16 == 0 && page_size > 0 &&
         shared_bytes(4, rank, rot_dim, 2) <= kSharedLimit;
}

// Floats of scratch a launch with `pieces` > 1 needs.
B200_API int64_t b200_latent_attention_mma_scratch(int num_seqs, int max_q_len, int heads, int rank, int pieces) {
  return pieces > 1 ? static_cast<int64_t>(num_seqs) * max_q_len * heads * pieces * (rank + 2) : 0;
}

// Requests first_seq .. first_seq + num_seqs of the step, each with up to max_q_len new tokens.
B200_API int b200_latent_attention_mma(const void* q_lat, int64_t q_lat_token, int64_t q_lat_head, const void* q_rot,
                                       const void* arena, const int* block_table, int max_pages, int num_pages, int page_size,
                                       const int* seq_q_start, const int* seq_q_len, const int* seq_kv_len, int first_seq,
                                       int num_seqs, int max_q_len, const float* sink, const void* gate, int64_t gate_ld,
                                       void* out, int64_t out_token, int64_t out_head, int heads, int rank, int rot_dim,
                                       float scale, int pieces, float* partial, int* err, cudaStream_t stream) {
  if (num_seqs <= 0 || max_q_len <= 0) return 0;
  B200_REQUIRE(b200_latent_attention_mma_supported(heads, rank, rot_dim, page_size), "latent_attention_mma: shape not taken");
  B200_REQUIRE(pieces >= 1 && pieces <= 65535 && (pieces == 1 || partial), "latent_attention_mma: bad split");
  B200_REQUIRE(num_seqs <= 65535, "latent_attention_mma: too many requests");
  const auto aligned = [](const void* ptr) { return reinterpret_cast<uintptr_t>(ptr) % 16 == 0; };
  B200_REQUIRE(aligned(q_lat) && aligned(q_rot) && aligned(arena) && q_lat_token % 8 == 0 && q_lat_head % 8 == 0 &&
                   out_token % 2 == 0 && out_head % 2 == 0 && reinterpret_cast<uintptr_t>(out) % 4 == 0,
               "latent_attention_mma: operands must be aligned to 16 bytes");
  LatentParams p;
  p.q_lat = static_cast<const __nv_bfloat16*>(q_lat), p.q_lat_token = q_lat_token, p.q_lat_head = q_lat_head;
  p.q_rot = static_cast<const __nv_bfloat16*>(q_rot), p.arena = static_cast<const __nv_bfloat16*>(arena);
  p.block_table = block_table, p.max_pages = max_pages, p.num_pages = num_pages, p.page_size = page_size;
  p.seq_q_start = seq_q_start, p.seq_q_len = seq_q_len, p.seq_kv_len = seq_kv_len, p.first_seq = first_seq;
  p.sink = sink, p.gate = static_cast<const __nv_bfloat16*>(gate), p.gate_ld = gate_ld;
  p.out = static_cast<__nv_bfloat16*>(out), p.out_token = out_token, p.out_head = out_head;
  p.partial = partial, p.rows_cap = max_q_len * heads;
  p.heads = heads, p.rank = rank, p.rot_dim = rot_dim, p.scale_log2 = scale * kLog2e, p.err = err;
  const int64_t rows = static_cast<int64_t>(max_q_len) * heads;
  const int rw = rows <= 16 ? 1 : (rows <= 32 ? 2 : 4);
  const dim3 grid(static_cast<unsigned>((rows + 16 * rw - 1) / (16 * rw)), num_seqs, pieces);
  // Two stages: measured on a B200 (12 heads, latent 512 + 64), a third stage changes nothing for prompt
  // portions (1.05 against 1.01 ms for three layers of 2,048 tokens) and costs single tokens their second
  // block per SM (72 against 55 us per layer for 8 requests of 2,048 keys).
  p.stages = 2;
  const size_t smem = shared_bytes(rw, rank, rot_dim, p.stages);
  int status = rw == 1 ? launch_for_rank<1>(p, grid, smem, stream)
                       : (rw == 2 ? launch_for_rank<2>(p, grid, smem, stream) : launch_for_rank<4>(p, grid, smem, stream));
  if (status != 0 || pieces == 1) return status;
  launch_kernel(latent_attention_merge_kernel, dim3(static_cast<unsigned>(rows), num_seqs), dim3(128), 0, stream, partial, pieces,
                p.rows_cap, rank, heads, first_seq, seq_q_start, seq_q_len, p.gate, gate_ld, p.out, out_token, out_head);
  return b200_check_launch("latent_attention_merge");
}
