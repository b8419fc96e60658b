// Attention over a cached latent on tensor cores (bfloat16 cache, mma.sync m16n8k16, 32-bit scores and sums).
//
// Every head attends over the same cached rows [c | k_rot] (Dk values, of which the first `rank` are also the
// "values"), so the 16 rows of an MMA are either 16 consecutive tokens of one request for one head (portions of
// prompts) or one token's 16 heads (single decoded tokens): TQ tokens x HB heads with TQ * HB = 16. One CTA of four
// warps per such group walks the keys in tiles of 64 positions:
//   the tile's rows come from the pages into shared memory (16-byte cp.async, zero-filled outside the group's key range);
//   warp w takes keys 16 w .. 16 w + 15: S = Q K^T over Dk, scale, per-row window and causal mask;
//   the row maximum over the four warps goes through shared memory; P = exp2(S - max) is written as bfloat16;
//   warp w owns rank / 4 of the output columns: O[:, its columns] = O * corr + P V with V the same shared tile.
// Portions of prompts with two heads or more run two to four heads to a CTA (four warps each) over the same key tiles,
// copied into two buffers in turn (`latent_attention_pair_kernel`).
// Row sums are kept per thread and added up at the end. The plain kernel (latent_attention.cu) serves the 32-bit
// path and the sizes this one refuses (Dk not a multiple of 16, rank not a multiple of 32 or above 512).
#include "common.cuh"
#include <math.h>
#include <stdlib.h>

namespace {

typedef __nv_bfloat16 bf16;
constexpr int KT = 64;   // keys per tile
constexpr int PAD = 8;   // bfloat16 values of padding per shared-memory row: ldmatrix rows fall into different banks
constexpr int PS = KT + PAD;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool valid) {
  int n = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(n) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_but_one() { asm volatile("cp.async.wait_group 1;" ::: "memory"); }
__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
      "{%0, %1, %2, %3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

struct Params {
  const float* qk;   // [rows, H, Dk] 32-bit: per head [query carried into the latent space | rotated part]
  float* out;        // [rows, H, rank]
  const bf16* pool;  // [n_blocks][bs][Dk]
  int n_blocks, bs;
  const int* positions;
  const int* seq_of_row;
  const int* tables;
  int table_stride;
  const int* tile_row0;   // portions: first row and row count of every group of up to TQ consecutive rows
  const int* tile_nrows;
  const int* rows;        // single tokens: the row of every group (null: group b is row b)
  int H, rank, Dk;
  float scale_log2;       // scale * log2(e)
  int window;
  const float* sink;      // (or null) per head: one more term exp(sink[head]) without a value in the denominator
  int TQ, HB;             // tokens x heads of a group, TQ * HB = 16
  int* err;
  // Single tokens with few groups: the key tiles of a group are dealt to n_splits CTAs (blockIdx.z), each leaves its
  // unnormalised sums, maximum and row sum, and `latent_merge_kernel` puts them together in split order.
  int n_splits;
  float* part_acc;        // [groups, head blocks, n_splits, 16, rank]
  float* part_ml;         // [groups, head blocks, n_splits, 16, 2]: maximum (of scores times log2 e), row sum
};

// NT8: most 8-column output tiles a warp owns (rank / 4 / 8 of them are used)
template <int NT8>
__global__ void __launch_bounds__(128)
latent_attention_mma_kernel(Params p) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int RS = p.Dk + PAD;  // row stride of Qs and Ks in values
  bf16* Qs = reinterpret_cast<bf16*>(smem_raw);
  bf16* Ks = Qs + 16 * RS;
  bf16* Ps = Ks + KT * RS;
  float* wmax = reinterpret_cast<float*>(Ps + 16 * PS);  // [4][16]
  float* wsum = wmax + 64;                               // [4][16]
  pdl_trigger();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  int row0, nrows;
  if (p.tile_row0) {
    row0 = p.tile_row0[blockIdx.x];
    nrows = p.tile_nrows[blockIdx.x];
  } else {
    row0 = p.rows ? p.rows[blockIdx.x] : (int)blockIdx.x;
    nrows = 1;
  }
  const int seq = p.seq_of_row[row0];
  if (seq < 0 || nrows <= 0) return;
  if (nrows > p.TQ) nrows = p.TQ;
  const int head0 = blockIdx.y * p.HB;
  const int P0 = p.positions[row0];
  const int Pmax = P0 + nrows - 1;
  const int lo_tile = (p.window > 0 && P0 - (p.window - 1) > 0) ? P0 - (p.window - 1) : 0;
  const int H = p.H, Dk = p.Dk, rank = p.rank;

  // the group's queries, as bfloat16
  for (int e = threadIdx.x; e < 16 * Dk; e += 128) {
    const int r = e / Dk, i = e - r * Dk;
    const int tok = r / p.HB, head = head0 + r % p.HB;
    float v = 0.f;
    if (tok < nrows && head < H) v = p.qk[((size_t)(row0 + tok) * H + head) * Dk + i];
    Qs[r * RS + i] = __float2bfloat16_rn(v);
  }
  // rows g and g + 8 of this thread
  int Pr[2], lor[2];
  bool rvalid[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int r = g + 8 * i;
    const int tok = r / p.HB, head = head0 + r % p.HB;
    rvalid[i] = tok < nrows && head < H;
    Pr[i] = P0 + tok;
    lor[i] = (p.window > 0 && Pr[i] - (p.window - 1) > 0) ? Pr[i] - (p.window - 1) : 0;
  }
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
  float acc[NT8][4];
#pragma unroll
  for (int i = 0; i < NT8; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
  const int DW = rank >> 2;      // output columns of a warp
  const int ntiles = DW >> 3;    // 8-column tiles of a warp
  const int* table = p.tables + (size_t)seq * p.table_stride;
  const int chunks = Dk >> 3;    // 16-byte pieces of a cache row
  const uint32_t qs_addr = smem_u32(Qs), ks_addr = smem_u32(Ks), ps_addr = smem_u32(Ps);
  // ldmatrix lane addresses: A operand (16 rows x 16 columns), B from rows that are keys, B transposed from rows
  // that are keys with the output columns along the row
  const int a_row = (lane & 7) + ((lane >> 3) & 1) * 8, a_col = (lane >> 4) * 8;
  const int b_key = (lane & 7) + (lane >> 4) * 8, b_col = ((lane >> 3) & 1) * 8;
  const int v_key = (lane & 7) + ((lane >> 3) & 1) * 8, v_col = (lane >> 4) * 8;

  int kt_first = (lo_tile / KT) * KT, kt_last = Pmax;
  if (p.n_splits > 1) {
    const int tiles = (Pmax / KT) - (lo_tile / KT) + 1;
    const int each = (tiles + p.n_splits - 1) / p.n_splits;
    kt_first += (int)blockIdx.z * each * KT;
    const int end = kt_first + each * KT - 1;
    kt_last = end < Pmax ? end : Pmax;
  }
  __syncthreads();  // the queries are written (a split without tiles goes straight to the end)
  for (int kt = kt_first; kt <= kt_last; kt += KT) {
    __syncthreads();  // the tile before is read to the end (and, the first time, the queries are written)
    {
      // two threads per key: one page lookup each, then the row's 16-byte pieces in turn with nothing between them
      const int j = threadIdx.x >> 1;
      const int kp = kt + j;
      bool valid = kp >= lo_tile && kp <= Pmax;
      const bf16* src = p.pool;
      if (valid) {
        const int blk = table[kp / p.bs];
        if (blk < 0 || blk >= p.n_blocks) {
          if (p.err) atomicExch(p.err, CUCA_ERR_BLOCK_RANGE);
          valid = false;
        } else {
          src = p.pool + ((size_t)blk * p.bs + (kp % p.bs)) * Dk;
        }
      }
      const uint32_t dst = ks_addr + (uint32_t)(j * RS) * 2;
      for (int ch = threadIdx.x & 1; ch < chunks; ch += 2) cp_async16(dst + ch * 16, valid ? src + ch * 8 : p.pool, valid);
    }
    cp_async_commit();
    cp_async_wait_all();
    __syncthreads();

    // S for this warp's 16 keys
    float s[2][4];
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) s[i][j] = 0.f;
    for (int k0 = 0; k0 < Dk; k0 += 16) {
      uint32_t a[4], b[4];
      ldsm_x4(a, qs_addr + (uint32_t)(a_row * RS + k0 + a_col) * 2);
      ldsm_x4(b, ks_addr + (uint32_t)((warp * 16 + b_key) * RS + k0 + b_col) * 2);
      mma_bf16(s[0], a, b[0], b[1]);
      mma_bf16(s[1], a, b[2], b[3]);
    }
    // scale and mask; s[nt][0..1]: row g, keys kbase + nt * 8 + 2 t + {0, 1}; s[nt][2..3]: row g + 8
    const int kbase = kt + warp * 16 + 2 * t;
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int i = j >> 1;
        const int kp = kbase + nt * 8 + (j & 1);
        const bool ok = rvalid[i] && kp >= lor[i] && kp <= Pr[i];
        s[nt][j] = ok ? s[nt][j] * p.scale_log2 : -INFINITY;
        mx[i] = fmaxf(mx[i], s[nt][j]);
      }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 1));
      mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 2));
    }
    if (t == 0) {
      wmax[warp * 16 + g] = mx[0];
      wmax[warp * 16 + g + 8] = mx[1];
    }
    __syncthreads();
    float corr[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int r = g + 8 * i;
      const float tm = fmaxf(fmaxf(wmax[r], wmax[16 + r]), fmaxf(wmax[32 + r], wmax[48 + r]));
      const float mn = fmaxf(m[i], tm);
      corr[i] = (mn == -INFINITY) ? 1.f : exp2f(m[i] - mn);
      m[i] = mn;
    }
    float ps[2] = {0.f, 0.f};
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
      float pv[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int i = j >> 1;
        pv[j] = (m[i] == -INFINITY) ? 0.f : exp2f(s[nt][j] - m[i]);
        ps[i] += pv[j];
      }
      const int col = warp * 16 + nt * 8 + 2 * t;
      *reinterpret_cast<uint32_t*>(Ps + g * PS + col) = pack_bf16(pv[0], pv[1]);
      *reinterpret_cast<uint32_t*>(Ps + (g + 8) * PS + col) = pack_bf16(pv[2], pv[3]);
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) l[i] = l[i] * corr[i] + ps[i];
#pragma unroll
    for (int n = 0; n < NT8; ++n) {
      acc[n][0] *= corr[0];
      acc[n][1] *= corr[0];
      acc[n][2] *= corr[1];
      acc[n][3] *= corr[1];
    }
    __syncthreads();  // P of all four warps is written

    // O[:, this warp's columns] += P V
#pragma unroll
    for (int kk = 0; kk < KT / 16; ++kk) {
      uint32_t a[4];
      ldsm_x4(a, ps_addr + (uint32_t)(a_row * PS + kk * 16 + a_col) * 2);
#pragma unroll
      for (int np = 0; np < NT8 / 2; ++np) {
        if (2 * np < ntiles) {
          const bool second = 2 * np + 1 < ntiles;
          const int col = warp * DW + np * 16 + (second ? v_col : 0);
          uint32_t b[4];
          ldsm_x4_trans(b, ks_addr + (uint32_t)((kk * 16 + v_key) * RS + col) * 2);
          mma_bf16(acc[2 * np], a, b[0], b[1]);
          if (second) mma_bf16(acc[2 * np + 1], a, b[2], b[3]);
        }
      }
    }
  }
  // row sums over the quad and over the warps
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    l[i] += __shfl_xor_sync(0xffffffffu, l[i], 1);
    l[i] += __shfl_xor_sync(0xffffffffu, l[i], 2);
  }
  __syncthreads();
  if (t == 0) {
    wsum[warp * 16 + g] = l[0];
    wsum[warp * 16 + g + 8] = l[1];
  }
  __syncthreads();
  if (p.n_splits > 1) {
    const size_t cell = ((size_t)blockIdx.x * gridDim.y + blockIdx.y) * p.n_splits + blockIdx.z;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int r = g + 8 * i;
      float* o = p.part_acc + (cell * 16 + r) * rank + warp * DW;
#pragma unroll
      for (int n = 0; n < NT8; ++n) {
        if (n < ntiles) {
          o[n * 8 + 2 * t] = acc[n][2 * i];
          o[n * 8 + 2 * t + 1] = acc[n][2 * i + 1];
        }
      }
      if (warp == 0 && t == 0) {
        p.part_ml[(cell * 16 + r) * 2] = m[i];
        p.part_ml[(cell * 16 + r) * 2 + 1] = wsum[r] + wsum[16 + r] + wsum[32 + r] + wsum[48 + r];
      }
    }
    return;
  }
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    if (!rvalid[i]) continue;
    const int r = g + 8 * i;
    float L = wsum[r] + wsum[16 + r] + wsum[32 + r] + wsum[48 + r];
    const int tok = r / p.HB, head = head0 + r % p.HB;
    if (p.sink && m[i] != -INFINITY) L += exp2f(p.sink[head] * 1.4426950408889634f - m[i]);  // (m in log2 units)
    const float inv = L > 0.f ? 1.f / L : 0.f;
    float* o = p.out + ((size_t)(row0 + tok) * H + head) * rank + warp * DW;
#pragma unroll
    for (int n = 0; n < NT8; ++n) {
      if (n < ntiles) {
        o[n * 8 + 2 * t] = acc[n][2 * i] * inv;
        o[n * 8 + 2 * t + 1] = acc[n][2 * i + 1] * inv;
      }
    }
  }
}

// Portions of prompts, HG heads per CTA (2 to 4): 4 HG warps, warps 4 a .. 4 a + 3 take head HG y + a of the same 16
// tokens, each four as in the kernel above. The heads read the same key tiles, and the tiles go into two buffers in
// turn, so tile t + 1 is on its way while tile t is worked on: 1 / HG of the traffic from L2 per head, more warps per SM
// than one head's four, and no wait for a whole tile between two tiles' arithmetic. The arithmetic of a row (tile
// order, sums) is the kernel's above.
template <int NT8, int HG>
__global__ void __launch_bounds__(128 * HG)
latent_attention_pair_kernel(Params p) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int RS = p.Dk + PAD;
  bf16* Qs = reinterpret_cast<bf16*>(smem_raw);               // [HG heads][16][RS]
  bf16* Ks = Qs + HG * 16 * RS;                                 // [2 buffers][KT][RS]
  bf16* Ps = Ks + 2 * KT * RS;                                 // [HG heads][16][PS]
  float* wmax = reinterpret_cast<float*>(Ps + HG * 16 * PS);    // [HG heads][4][16]
  float* wsum = wmax + HG * 64;                                   // [HG heads][4][16]
  pdl_trigger();
  pdl_wait();
  const int grp = threadIdx.x >> 7, tid = threadIdx.x & 127;
  const int warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;
  const int row0 = p.tile_row0[blockIdx.x];
  int nrows = p.tile_nrows[blockIdx.x];
  const int seq = p.seq_of_row[row0];
  if (seq < 0 || nrows <= 0) return;  // (the same for every thread of the block)
  if (nrows > 16) nrows = 16;
  const int head = blockIdx.y * HG + grp;
  const bool head_ok = head < p.H;
  const int P0 = p.positions[row0];
  const int Pmax = P0 + nrows - 1;
  const int lo_tile = (p.window > 0 && P0 - (p.window - 1) > 0) ? P0 - (p.window - 1) : 0;
  const int H = p.H, Dk = p.Dk, rank = p.rank;
  bf16* Qg = Qs + grp * 16 * RS;
  bf16* Pg = Ps + grp * 16 * PS;
  float* wmaxg = wmax + grp * 64;
  float* wsumg = wsum + grp * 64;

  for (int e = tid; e < 16 * Dk; e += 128) {  // this head's queries, as bfloat16
    const int r = e / Dk, i = e - r * Dk;
    float v = 0.f;
    if (r < nrows && head_ok) v = p.qk[((size_t)(row0 + r) * H + head) * Dk + i];
    Qg[r * RS + i] = __float2bfloat16_rn(v);
  }
  int Pr[2], lor[2];
  bool rvalid[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int r = g + 8 * i;
    rvalid[i] = r < nrows && head_ok;
    Pr[i] = P0 + r;
    lor[i] = (p.window > 0 && Pr[i] - (p.window - 1) > 0) ? Pr[i] - (p.window - 1) : 0;
  }
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
  float acc[NT8][4];
#pragma unroll
  for (int i = 0; i < NT8; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
  const int DW = rank >> 2;
  const int ntiles = DW >> 3;
  const int* table = p.tables + (size_t)seq * p.table_stride;
  const int chunks = Dk >> 3;
  const uint32_t qs_addr = smem_u32(Qg), ks_addr = smem_u32(Ks), ps_addr = smem_u32(Pg);
  const int a_row = (lane & 7) + ((lane >> 3) & 1) * 8, a_col = (lane >> 4) * 8;
  const int b_key = (lane & 7) + (lane >> 4) * 8, b_col = ((lane >> 3) & 1) * 8;
  const int v_key = (lane & 7) + ((lane >> 3) & 1) * 8, v_col = (lane >> 4) * 8;

  // 2 HG threads per key: one page lookup each, then the row's 16-byte pieces in turn
  constexpr int TPK = 2 * HG;
  auto load_tile = [&](int kt, int buf) {
    const int j = threadIdx.x / TPK;
    const int kp = kt + j;
    bool valid = kp >= lo_tile && kp <= Pmax;
    const bf16* src = p.pool;
    if (valid) {
      const int blk = table[kp / p.bs];
      if (blk < 0 || blk >= p.n_blocks) {
        if (p.err) atomicExch(p.err, CUCA_ERR_BLOCK_RANGE);
        valid = false;
      } else {
        src = p.pool + ((size_t)blk * p.bs + (kp % p.bs)) * Dk;
      }
    }
    const uint32_t dst = ks_addr + (uint32_t)((buf * KT + j) * RS) * 2;
    for (int ch = threadIdx.x % TPK; ch < chunks; ch += TPK) cp_async16(dst + ch * 16, valid ? src + ch * 8 : p.pool, valid);
    cp_async_commit();
  };

  const int kt_first = (lo_tile / KT) * KT;
  load_tile(kt_first, 0);
  int buf = 0;
  for (int kt = kt_first; kt <= Pmax; kt += KT, buf ^= 1) {
    if (kt + KT <= Pmax) {
      load_tile(kt + KT, buf ^ 1);  // (that buffer was read to the end before the barrier that closed the last round)
      cp_async_wait_but_one();
    } else {
      cp_async_wait_all();
    }
    __syncthreads();  // tile kt is there for every thread (and, the first time, the queries are written)
    const uint32_t kb = ks_addr + (uint32_t)(buf * KT * RS) * 2;

    float s[2][4];
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) s[i][j] = 0.f;
    for (int k0 = 0; k0 < Dk; k0 += 16) {
      uint32_t a[4], b[4];
      ldsm_x4(a, qs_addr + (uint32_t)(a_row * RS + k0 + a_col) * 2);
      ldsm_x4(b, kb + (uint32_t)((warp * 16 + b_key) * RS + k0 + b_col) * 2);
      mma_bf16(s[0], a, b[0], b[1]);
      mma_bf16(s[1], a, b[2], b[3]);
    }
    const int kbase = kt + warp * 16 + 2 * t;
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int i = j >> 1;
        const int kp = kbase + nt * 8 + (j & 1);
        const bool ok = rvalid[i] && kp >= lor[i] && kp <= Pr[i];
        s[nt][j] = ok ? s[nt][j] * p.scale_log2 : -INFINITY;
        mx[i] = fmaxf(mx[i], s[nt][j]);
      }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 1));
      mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 2));
    }
    if (t == 0) {
      wmaxg[warp * 16 + g] = mx[0];
      wmaxg[warp * 16 + g + 8] = mx[1];
    }
    __syncthreads();
    float corr[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int r = g + 8 * i;
      const float tm = fmaxf(fmaxf(wmaxg[r], wmaxg[16 + r]), fmaxf(wmaxg[32 + r], wmaxg[48 + r]));
      const float mn = fmaxf(m[i], tm);
      corr[i] = (mn == -INFINITY) ? 1.f : exp2f(m[i] - mn);
      m[i] = mn;
    }
    float ps[2] = {0.f, 0.f};
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
      float pv[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int i = j >> 1;
        pv[j] = (m[i] == -INFINITY) ? 0.f : exp2f(s[nt][j] - m[i]);
        ps[i] += pv[j];
      }
      const int col = warp * 16 + nt * 8 + 2 * t;
      *reinterpret_cast<uint32_t*>(Pg + g * PS + col) = pack_bf16(pv[0], pv[1]);
      *reinterpret_cast<uint32_t*>(Pg + (g + 8) * PS + col) = pack_bf16(pv[2], pv[3]);
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) l[i] = l[i] * corr[i] + ps[i];
#pragma unroll
    for (int n = 0; n < NT8; ++n) {
      acc[n][0] *= corr[0];
      acc[n][1] *= corr[0];
      acc[n][2] *= corr[1];
      acc[n][3] *= corr[1];
    }
    __syncthreads();  // P of this head's four warps is written

#pragma unroll
    for (int kk = 0; kk < KT / 16; ++kk) {
      uint32_t a[4];
      ldsm_x4(a, ps_addr + (uint32_t)(a_row * PS + kk * 16 + a_col) * 2);
#pragma unroll
      for (int np = 0; np < NT8 / 2; ++np) {
        if (2 * np < ntiles) {
          const bool second = 2 * np + 1 < ntiles;
          const int col = warp * DW + np * 16 + (second ? v_col : 0);
          uint32_t b[4];
          ldsm_x4_trans(b, kb + (uint32_t)((kk * 16 + v_key) * RS + col) * 2);
          mma_bf16(acc[2 * np], a, b[0], b[1]);
          if (second) mma_bf16(acc[2 * np + 1], a, b[2], b[3]);
        }
      }
    }
    __syncthreads();  // the tile, the maxima and P are read to the end: the next round may overwrite them
  }
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    l[i] += __shfl_xor_sync(0xffffffffu, l[i], 1);
    l[i] += __shfl_xor_sync(0xffffffffu, l[i], 2);
  }
  if (t == 0) {
    wsumg[warp * 16 + g] = l[0];
    wsumg[warp * 16 + g + 8] = l[1];
  }
  __syncthreads();
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    if (!rvalid[i]) continue;
    const int r = g + 8 * i;
    float L = wsumg[r] + wsumg[16 + r] + wsumg[32 + r] + wsumg[48 + r];
    if (p.sink && m[i] != -INFINITY) L += exp2f(p.sink[head] * 1.4426950408889634f - m[i]);  // (m in log2 units)
    const float inv = L > 0.f ? 1.f / L : 0.f;
    float* o = p.out + ((size_t)(row0 + r) * H + head) * rank + warp * DW;
#pragma unroll
    for (int n = 0; n < NT8; ++n) {
      if (n < ntiles) {
        o[n * 8 + 2 * t] = acc[n][2 * i] * inv;
        o[n * 8 + 2 * t + 1] = acc[n][2 * i + 1] * inv;
      }
    }
  }
}

// One block per (group, head block, row of 16): out = sum_z acc_z 2^(m_z - M) / sum_z l_z 2^(m_z - M), z in order
// (up to 64 splits).
__global__ void latent_merge_kernel(const float* __restrict__ part_acc, const float* __restrict__ part_ml,
                                    float* __restrict__ out, const int* __restrict__ rows,
                                    const int* __restrict__ seq_of_row, int n_splits, int H, int rank,
                                    const float* __restrict__ sink) {
  pdl_trigger();
  pdl_wait();
  const int grp = blockIdx.x, hb = blockIdx.y, r = blockIdx.z;
  const int row = rows ? rows[grp] : grp;
  const int head = hb * 16 + r;
  if (head >= H || seq_of_row[row] < 0) return;
  const size_t cell0 = ((size_t)grp * gridDim.y + hb) * n_splits;
  __shared__ float wz[64];  // every split's weight 2^(m_z - M) / L, worked out once by the first warp
  if (threadIdx.x < 32) {
    float mz[2], lz[2];
    float M = -INFINITY;
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      const int z = threadIdx.x + 32 * k;
      mz[k] = z < n_splits ? part_ml[((cell0 + z) * 16 + r) * 2] : -INFINITY;
      lz[k] = z < n_splits ? part_ml[((cell0 + z) * 16 + r) * 2 + 1] : 0.f;
      M = fmaxf(M, mz[k]);
    }
    M = warp_max(M);
    float e[2], L = 0.f;
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      e[k] = mz[k] == -INFINITY ? 0.f : exp2f(mz[k] - M);
      L += lz[k] * e[k];
    }
    L = warp_sum(L);
    if (sink && M != -INFINITY) L += exp2f(sink[head] * 1.4426950408889634f - M);
    const float inv = L > 0.f ? 1.f / L : 0.f;
    wz[threadIdx.x] = e[0] * inv;
    wz[threadIdx.x + 32] = e[1] * inv;
  }
  __syncthreads();
  for (int c = threadIdx.x; c < rank; c += blockDim.x) {
    float a = 0.f;
    for (int z = 0; z < n_splits; ++z) a = fmaf(part_acc[((cell0 + z) * 16 + r) * rank + c], wz[z], a);
    out[((size_t)row * H + head) * rank + c] = a;
  }
}

size_t smem_bytes(int Dk) {
  return (size_t)(16 + KT) * (Dk + PAD) * sizeof(bf16) + (size_t)16 * PS * sizeof(bf16) + 2 * 64 * sizeof(float);
}

template <int NT8>
int launch(const Params& p, int n_groups, int head_blocks, cudaStream_t stream) {
  const size_t smem = smem_bytes(p.Dk);
  static size_t configured = 0;
  if (smem > configured) {
    cudaError_t e = cudaFuncSetAttribute(latent_attention_mma_kernel<NT8>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)smem);
    if (e != cudaSuccess) {
      cuca_set_error("latent_attention_mma: %zu bytes of shared memory refused: %s", smem, cudaGetErrorString(e));
      return 2;
    }
    configured = smem;
  }
  cuca_launch(latent_attention_mma_kernel<NT8>, dim3(n_groups, head_blocks, p.n_splits), dim3(128), smem, stream,
              true, p);
  return 0;
}

size_t pair_smem_bytes(int Dk, int hg) {
  return (size_t)(hg * 16 + 2 * KT) * (Dk + PAD) * sizeof(bf16) + (size_t)hg * 16 * PS * sizeof(bf16) +
         (size_t)hg * 128 * sizeof(float);
}

template <int NT8, int HG>
int launch_pair(const Params& p, int n_groups, cudaStream_t stream) {
  const size_t smem = pair_smem_bytes(p.Dk, HG);
  static size_t configured = 0;
  if (smem > configured) {
    cudaError_t e = cudaFuncSetAttribute(latent_attention_pair_kernel<NT8, HG>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) {
      cuca_set_error("latent_attention_mma: %zu bytes of shared memory refused: %s", smem, cudaGetErrorString(e));
      return 2;
    }
    configured = smem;
  }
  cuca_launch(latent_attention_pair_kernel<NT8, HG>, dim3(n_groups, (p.H + HG - 1) / HG, 1), dim3(128 * HG), smem,
              stream, true, p);
  return 0;
}

// How many heads of a portion's 16 tokens share a CTA (0: the one-head kernel): as many of 4, 3, 2 as the heads and
// shared memory allow (CUCA_LATENT_PAIR=0: never; =2, 3, 4: at most that many; a measuring aid).
int heads_per_cta(const Params& p, bool portions) {
  static const int most = getenv("CUCA_LATENT_PAIR") ? atoi(getenv("CUCA_LATENT_PAIR")) : 4;
  if (!portions) return 0;
  for (int hg = most < 4 ? most : 4; hg >= 2; --hg)
    if (p.H >= hg && pair_smem_bytes(p.Dk, hg) <= 227 * 1024) return hg;
  return 0;
}

template <int NT8>
int launch_pair_by_heads(const Params& p, int hg, int n_groups, cudaStream_t stream) {
  if (hg == 4) return launch_pair<NT8, 4>(p, n_groups, stream);
  if (hg == 3) return launch_pair<NT8, 3>(p, n_groups, stream);
  return launch_pair<NT8, 2>(p, n_groups, stream);
}

}  // namespace

// Whether the tensor-core form takes these sizes (the cache must be bfloat16).
CUCA_API int cuca_latent_attention_mma_supported(int rank, int Dk) {
  return Dk % 16 == 0 && rank % 32 == 0 && rank >= 32 && rank <= 512 && rank <= Dk && smem_bytes(Dk) <= 227 * 1024;
}

// Groups of rows: with tile_row0/tile_nrows, `n_groups` runs of up to 16 consecutive rows of one request (one head
// per CTA); without, `n_groups` single rows (`rows`, or 0..n_groups-1 when null) with 16 heads per CTA.
// sink (or null): 32-bit, one number per head: one more term exp(sink[head]) without a value in every denominator.
CUCA_API int cuca_latent_attention_mma_s(const float* qk, float* out, const void* pool, int n_blocks, int bs,
                                         const int* positions, const int* seq_of_row, const int* tables,
                                         int table_stride, const int* tile_row0, const int* tile_nrows, const int* rows,
                                         int n_groups, int H, int rank, int Dk, float scale, int window,
                                         const float* sink, int n_splits, float* part_acc, float* part_ml, int* err,
                                         cudaStream_t stream) {
  if (n_groups == 0) return 0;
  CUCA_REQUIRE(cuca_latent_attention_mma_supported(rank, Dk), "latent_attention_mma: sizes rank=%d Dk=%d are not taken",
               rank, Dk);
  Params p;
  p.qk = qk; p.out = out; p.pool = (const bf16*)pool; p.n_blocks = n_blocks; p.bs = bs; p.positions = positions;
  p.seq_of_row = seq_of_row; p.tables = tables; p.table_stride = table_stride; p.tile_row0 = tile_row0;
  p.tile_nrows = tile_nrows; p.rows = rows; p.H = H; p.rank = rank; p.Dk = Dk;
  p.scale_log2 = scale * 1.4426950408889634f; p.window = window; p.err = err; p.sink = sink;
  p.n_splits = (tile_row0 == nullptr && n_splits > 1 && part_acc && part_ml) ? n_splits : 1;
  p.part_acc = part_acc; p.part_ml = part_ml;
  CUCA_REQUIRE(p.n_splits <= 64, "latent_attention_mma: %d splits exceed 64", n_splits);
  const bool portions = tile_row0 != nullptr;
  p.TQ = portions ? 16 : 1;
  p.HB = portions ? 1 : 16;
  const int head_blocks = (H + p.HB - 1) / p.HB;
  CUCA_REQUIRE(head_blocks <= 65535, "latent_attention_mma: %d heads exceed the launch limit", H);
  const int ntiles = rank / 32;
  int rc;
  if (const int hg = heads_per_cta(p, portions)) {
    CUCA_REQUIRE((H + hg - 1) / hg <= 65535, "latent_attention_mma: %d heads exceed the launch limit", H);
    if (ntiles <= 4) rc = launch_pair_by_heads<4>(p, hg, n_groups, stream);
    else if (ntiles <= 8) rc = launch_pair_by_heads<8>(p, hg, n_groups, stream);
    else rc = launch_pair_by_heads<16>(p, hg, n_groups, stream);
    if (rc) return rc;
    CUCA_CHECK_LAUNCH("latent_attention_mma");
    return 0;
  }
  if (ntiles <= 4) rc = launch<4>(p, n_groups, head_blocks, stream);
  else if (ntiles <= 8) rc = launch<8>(p, n_groups, head_blocks, stream);
  else rc = launch<16>(p, n_groups, head_blocks, stream);
  if (rc) return rc;
  CUCA_CHECK_LAUNCH("latent_attention_mma");
  if (p.n_splits > 1) {
    cuca_launch(latent_merge_kernel, dim3(n_groups, head_blocks, 16), dim3(128), 0, stream, true,
                (const float*)part_acc, (const float*)part_ml, out, rows, seq_of_row, p.n_splits, H, rank, sink);
    CUCA_CHECK_LAUNCH("latent_merge");
  }
  return 0;
}

CUCA_API int cuca_latent_attention_mma(const float* qk, float* out, const void* pool, int n_blocks, int bs,
                                       const int* positions, const int* seq_of_row, const int* tables,
                                       int table_stride, const int* tile_row0, const int* tile_nrows, const int* rows,
                                       int n_groups, int H, int rank, int Dk, float scale, int window, int n_splits,
                                       float* part_acc, float* part_ml, int* err, cudaStream_t stream) {
  return cuca_latent_attention_mma_s(qk, out, pool, n_blocks, bs, positions, seq_of_row, tables, table_stride, tile_row0,
                                     tile_nrows, rows, n_groups, H, rank, Dk, scale, window, nullptr, n_splits, part_acc,
                                     part_ml, err, stream);
}
