// Paged causal grouped-query attention, plain form: one warp per (row, query
// head), keys in tiles of 32 absolute positions with an online softmax. It
// serves the true 32-bit path and is the fall-back of the bfloat16 path for
// head sizes its tensor-core kernels refuse. A row's arithmetic depends only
// on its own position and keys: tiles start at multiples of 32 key positions,
// so cutting a prompt or batching it differently gives the same bits.
#include "common.cuh"
#include <math.h>

namespace {

// VC: runs of 32 value columns a lane accumulates (value heads of up to 32 VC values)
template <typename T, int VC>
__global__ void __launch_bounds__(128)
attention_generic_kernel(const T* __restrict__ q, int q_stride, T* __restrict__ out, int out_stride,
                         const T* __restrict__ kpool, const T* __restrict__ vpool, int n_blocks, int bs,
                         const int* __restrict__ positions, const int* __restrict__ seq_of_row,
                         const int* __restrict__ tables, int table_stride, int nh, int nkv, int d, int dv,
                         float scale, int window, float softcap, int sink, const float* __restrict__ sink_val,
                         int* err) {
  extern __shared__ float qs[];  // [4][d]
  pdl_trigger();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row = blockIdx.y;
  const int head = blockIdx.x * 4 + warp;
  const int seq = seq_of_row[row];
  if (seq < 0 || head >= nh) return;
  const int P = positions[row];
  const int kvh = head / (nh / nkv);
  float* qv = qs + warp * d;
  const T* qrow = q + (size_t)row * q_stride + (size_t)head * d;
  for (int i = lane; i < d; i += 32) qv[i] = to_f32(qrow[i]);
  __syncwarp();

  int lo = 0;
  if (window > 0 && P - (window - 1) > 0) lo = P - (window - 1);
  float m = -INFINITY, l = 0.f;
  float acc[VC];
#pragma unroll
  for (int c = 0; c < VC; ++c) acc[c] = 0.f;
  const int* table = tables + (size_t)seq * table_stride;

  for (int t0 = (lo / 32) * 32; t0 <= P; t0 += 32) {
    int kp = t0 + lane;
    bool valid = kp >= lo && kp <= P;
    long long base = -1;  // this key's row number in the pools (key rows of d values, value rows of dv)
    if (valid) {
      int blk = table[kp / bs];
      if (blk < 0 || blk >= n_blocks) {
        if (err) atomicExch(err, CUCA_ERR_BLOCK_RANGE);
        valid = false;
      } else {
        base = ((long long)blk * nkv + kvh) * bs + (kp % bs);
      }
    }
    float s = -INFINITY;
    if (valid) {
      const T* kr = kpool + base * d;
      float dot = 0.f;
      for (int i = 0; i < d; ++i) dot = fmaf(qv[i], to_f32(kr[i]), dot);
      s = dot * scale;
      if (softcap > 0.f) s = softcap * tanhf(s / softcap);  // a smooth cap on the score
    }
    float m_new = fmaxf(m, warp_max(s));
    if (m_new == -INFINITY) continue;  // a tile with no readable key
    float p = valid ? expf(s - m_new) : 0.f;
    float corr = expf(m - m_new);
    l = l * corr + warp_sum(p);
#pragma unroll
    for (int c = 0; c < VC; ++c) acc[c] *= corr;
    for (int j = 0; j < 32; ++j) {
      float pj = __shfl_sync(0xffffffffu, p, j);
      long long bj = __shfl_sync(0xffffffffu, base, j);
      if (bj < 0) continue;
      const T* vr = vpool + bj * dv;
#pragma unroll
      for (int c = 0; c < VC; ++c) {
        int dim = c * 32 + lane;
        if (dim < dv) acc[c] = fmaf(pj, to_f32(vr[dim]), acc[c]);
      }
    }
    m = m_new;
  }
  if (sink) {  // one more term in the denominator: a key of score 0 (or of the head's stored score) that has no value
    const float s0 = sink_val ? sink_val[head] : 0.f;
    const float m_new = fmaxf(m, s0);
    const float corr = expf(m - m_new);
    l = l * corr + expf(s0 - m_new);
#pragma unroll
    for (int c = 0; c < VC; ++c) acc[c] *= corr;
  }
  float inv = l > 0.f ? 1.f / l : 0.f;
  T* o = out + (size_t)row * out_stride + (size_t)head * dv;
#pragma unroll
  for (int c = 0; c < VC; ++c) {
    int dim = c * 32 + lane;
    if (dim < dv) o[dim] = from_f32<T>(acc[c] * inv);
  }
}

}  // namespace

// The largest head size any attention kernel of this library takes (the plain kernel's; the tensor-core forms take
// fewer). A part asks at construction, so that a model with larger heads is refused when it is built, not at its
// first step.
CUCA_API int cuca_attention_max_head_dim() { return 256; }

// q: rows of `q_stride` elements whose first nh*d hold the (rotated) query
// heads; out: [n_rows, out_stride] with nh heads of dv values; key pool [n_blocks][nkv][bs][d], value pool
// [n_blocks][nkv][bs][dv]. Row r is at position positions[r] of sequence seq_of_row[r] (< 0: padding, skipped) and
// sees keys max(0, P - window + 1)..P of that sequence (window 0: all). softcap c > 0: a score s becomes
// c tanh(s / c). sink: the softmax's denominator holds one more term, exp(0), or with sink_val (32-bit, one number per
// query head) exp(sink_val[head]): a score that is neither scaled nor capped.
CUCA_API int cuca_attention_generic_sv(const void* q, int q_stride, void* out, int out_stride, int dtype,
                                      const void* kpool, const void* vpool, int n_blocks, int bs,
                                      const int* positions, const int* seq_of_row, const int* tables,
                                      int table_stride, int n_rows, int nh, int nkv, int d, int dv, float scale,
                                      int window, float softcap, int sink, const float* sink_val, int* err,
                                      cudaStream_t stream) {
  if (n_rows == 0) return 0;
  CUCA_REQUIRE(d > 0 && d <= cuca_attention_max_head_dim(), "attention: head size %d is outside 1..%d", d, cuca_attention_max_head_dim());
  CUCA_REQUIRE(dv > 0 && dv <= 2 * cuca_attention_max_head_dim(), "attention: value size %d is outside 1..%d", dv,
               2 * cuca_attention_max_head_dim());
  CUCA_REQUIRE(nkv > 0 && nh % nkv == 0, "attention: %d query heads do not group over %d key heads", nh, nkv);
  CUCA_REQUIRE(n_rows <= 65535, "attention: %d rows in one step exceed the launch limit 65535", n_rows);
  dim3 grid((nh + 3) / 4, n_rows);
  size_t smem = (size_t)4 * d * sizeof(float);
#define AG(T, VC)                                                                                                  \
  cuca_launch(attention_generic_kernel<T, VC>, grid, dim3(128), smem, stream, true, (const T*)q, q_stride, (T*)out, \
              out_stride, (const T*)kpool, (const T*)vpool, n_blocks, bs, positions, seq_of_row, tables,            \
              table_stride, nh, nkv, d, dv, scale, window, softcap, sink, sink_val, err)
  if (dtype == CUCA_F32) {
    if (dv <= 256) AG(float, 8); else AG(float, 16);
  } else if (dtype == CUCA_BF16) {
    if (dv <= 256) AG(__nv_bfloat16, 8); else AG(__nv_bfloat16, 16);
  } else {
    CUCA_REQUIRE(false, "attention: unknown dtype %d", dtype);
  }
#undef AG
  CUCA_CHECK_LAUNCH("attention_generic");
  return 0;
}

CUCA_API int cuca_attention_generic_s(const void* q, int q_stride, void* out, int out_stride, int dtype,
                                      const void* kpool, const void* vpool, int n_blocks, int bs,
                                      const int* positions, const int* seq_of_row, const int* tables,
                                      int table_stride, int n_rows, int nh, int nkv, int d, int dv, float scale,
                                      int window, float softcap, int sink, int* err, cudaStream_t stream) {
  return cuca_attention_generic_sv(q, q_stride, out, out_stride, dtype, kpool, vpool, n_blocks, bs, positions, seq_of_row,
                                  tables, table_stride, n_rows, nh, nkv, d, dv, scale, window, softcap, sink, nullptr,
                                  err, stream);
}

CUCA_API int cuca_attention_generic_v(const void* q, int q_stride, void* out, int out_stride, int dtype,
                                      const void* kpool, const void* vpool, int n_blocks, int bs,
                                      const int* positions, const int* seq_of_row, const int* tables,
                                      int table_stride, int n_rows, int nh, int nkv, int d, int dv, float scale,
                                      int window, int* err, cudaStream_t stream) {
  return cuca_attention_generic_s(q, q_stride, out, out_stride, dtype, kpool, vpool, n_blocks, bs, positions, seq_of_row,
                                  tables, table_stride, n_rows, nh, nkv, d, dv, scale, window, 0.f, 0, err, stream);
}

CUCA_API int cuca_attention_generic(const void* q, int q_stride, void* out, int out_stride, int dtype,
                                    const void* kpool, const void* vpool, int n_blocks, int bs,
                                    const int* positions, const int* seq_of_row, const int* tables,
                                    int table_stride, int n_rows, int nh, int nkv, int d, float scale,
                                    int window, int* err, cudaStream_t stream) {
  return cuca_attention_generic_v(q, q_stride, out, out_stride, dtype, kpool, vpool, n_blocks, bs, positions,
                                  seq_of_row, tables, table_stride, n_rows, nh, nkv, d, d, scale, window, err, stream);
}

// ---------------------------------------------------------------- rotation and the paged write, general form
// qkv: rows of `ld` values: nh query heads of d at column 0, nkv key heads of d at k_col, nkv value heads of dv at
// v_col. The first `rot` values of every q and k head are rotated by the row's position, in pairs (i, i + rot/2)
// (pairs 0) or (2i, 2i + 1) (pairs 1); q in place, k and v go to the position's page. v_split r > 1: the value pool
// is r slabs [n_blocks][nkv][bs][dv / r], slab j holding values j dv/r .. (j+1) dv/r - 1 of every head (each slab is
// then a value pool of narrower heads for the kernels that want values as wide as keys). dv_src < dv: a row's value
// heads hold dv_src values and the pool's dv: the rest of a pool row is written as zeros (values padded to a
// multiple of the key size for those kernels).
namespace {
template <typename T>
__global__ void __launch_bounds__(256)
rope_store_general_kernel(T* __restrict__ qkv, int ld, int k_col, int v_col, const int* __restrict__ positions,
                          const int* __restrict__ seq_of_row, const int* __restrict__ tables, int table_stride,
                          const float* __restrict__ cos_t, const float* __restrict__ sin_t, int table_rows, int rot,
                          int pairs, T* __restrict__ kpool, T* __restrict__ vpool, int n_blocks, int bs, int nh,
                          int nkv, int d, int dv, int v_split, int dv_src, int* err) {
  pdl_trigger();
  pdl_wait();
  const int row = blockIdx.x;
  const int seq = seq_of_row[row];
  if (seq < 0) return;
  const int pos = positions[row];
  const int half = rot / 2;
  T* base = qkv + (size_t)row * ld;
  long long page_row = -1;
  if (nkv > 0) {
    int blk = pos >= 0 ? tables[(size_t)seq * table_stride + pos / bs] : -1;
    if (blk < 0 || blk >= n_blocks) {
      if (threadIdx.x == 0 && err) atomicExch(err, CUCA_ERR_BLOCK_RANGE);
    } else {
      page_row = (long long)blk * nkv * bs + (pos % bs);
    }
  }
  const bool in_table = pos >= 0 && pos < table_rows;
  if (!in_table && half > 0 && threadIdx.x == 0 && err) atomicExch(err, CUCA_ERR_TOKEN_RANGE);
  const float* cr = cos_t + (size_t)(in_table ? pos : 0) * half;
  const float* sr = sin_t + (size_t)(in_table ? pos : 0) * half;
  const int per_head = half + (d - rot);
  for (int idx = threadIdx.x; idx < (nh + nkv) * per_head; idx += blockDim.x) {
    const int head = idx / per_head, i = idx % per_head;
    const bool is_k = head >= nh;
    T* src = is_k ? base + k_col + (size_t)(head - nh) * d : base + (size_t)head * d;
    T* dst = src;
    if (is_k) {
      if (page_row < 0) continue;
      dst = kpool + (page_row + (long long)(head - nh) * bs) * d;
    }
    if (i < half) {
      const int ia = pairs ? 2 * i : i, ib = pairs ? 2 * i + 1 : i + half;
      const float c = in_table ? cr[i] : 1.f, sn = in_table ? sr[i] : 0.f;
      const float a = to_f32(src[ia]), b = to_f32(src[ib]);
      dst[ia] = from_f32<T>(a * c - b * sn);
      dst[ib] = from_f32<T>(b * c + a * sn);
    } else if (is_k) {
      const int e = rot + (i - half);
      dst[e] = src[e];
    }
  }
  if (nkv > 0 && page_row >= 0) {
    const T* vsrc = base + v_col;
    const int ds = dv / v_split;
    const long long slab_rows = (long long)n_blocks * nkv * bs;
    for (int idx = threadIdx.x; idx < nkv * dv; idx += blockDim.x) {
      const int kvh = idx / dv, e = idx % dv;
      vpool[((e / ds) * slab_rows + page_row + (long long)kvh * bs) * ds + e % ds] =
          e < dv_src ? vsrc[(size_t)kvh * dv_src + e] : from_f32<T>(0.f);
    }
  }
}
}  // namespace

CUCA_API int cuca_rope_store_general(void* qkv, int dtype, int ld, int k_col, int v_col, const int* positions,
                                     const int* seq_of_row, const int* tables, int table_stride, const float* cos_t,
                                     const float* sin_t, int table_rows, int rot, int pairs, void* kpool, void* vpool,
                                     int n_blocks, int bs, int n_rows, int nh, int nkv, int d, int dv, int v_split,
                                     int dv_src, int* err, cudaStream_t stream) {
  if (n_rows == 0) return 0;
  if (dv_src <= 0) dv_src = dv;
  CUCA_REQUIRE(dv_src <= dv, "rope_store: rows with %d values a head do not fit a pool of %d", dv_src, dv);
  CUCA_REQUIRE(rot >= 0 && rot <= d && rot % 2 == 0, "rope_store: rotary size %d does not fit head size %d", rot, d);
  CUCA_REQUIRE(bs > 0 && nh > 0 && nkv >= 0 && d > 0 && dv > 0, "rope_store: bad sizes");
  CUCA_REQUIRE(v_split >= 1 && dv % v_split == 0, "rope_store: %d slabs do not divide value size %d", v_split, dv);
  if (dtype == CUCA_F32)
    cuca_launch(rope_store_general_kernel<float>, dim3(n_rows), dim3(256), 0, stream, true, (float*)qkv, ld, k_col,
                v_col, positions, seq_of_row, tables, table_stride, cos_t, sin_t, table_rows, rot, pairs, (float*)kpool,
                (float*)vpool, n_blocks, bs, nh, nkv, d, dv, v_split, dv_src, err);
  else if (dtype == CUCA_BF16)
    cuca_launch(rope_store_general_kernel<__nv_bfloat16>, dim3(n_rows), dim3(256), 0, stream, true, (__nv_bfloat16*)qkv,
                ld, k_col, v_col, positions, seq_of_row, tables, table_stride, cos_t, sin_t, table_rows, rot, pairs,
                (__nv_bfloat16*)kpool, (__nv_bfloat16*)vpool, n_blocks, bs, nh, nkv, d, dv, v_split, dv_src, err);
  else
    CUCA_REQUIRE(false, "rope_store: unknown dtype %d", dtype);
  CUCA_CHECK_LAUNCH("rope_store_general");
  return 0;
}

// ---------------------------------------------------------------- head norms, rotation and the paged write
// As above, with norms per head in 32-bit before the rotation: a q head becomes q / rms(q) * q_norm (k alike with
// k_norm; a null weight: no norm), and with v_norm a v head becomes v / rms(v) (no weight) before it is kept. T is the
// rows' type (a 32-bit projection result may feed 16-bit pools: TP); q is written in place when q_out is null, else to
// q_out [rows, nh d] of the pools' type. A warp per head.
// whole != 0: the norm is over the whole projection instead, all heads at once: q / rms(q over its nh d values) times
// q_norm [nh d], k alike over its nkv d values with k_norm [nkv d] (v_norm is not combined with it).
// qt_every > 0: the query of a row at position p is multiplied by 1 + qt_coef ln(floor((p + 1) / qt_every) + 1), after
// norm and rotation.
namespace {
template <typename T, typename TP>
__global__ void __launch_bounds__(256)
norm_rope_store_kernel(T* __restrict__ qkv, int ld, int k_col, int v_col, TP* __restrict__ q_out,
                       const int* __restrict__ positions, const int* __restrict__ seq_of_row,
                       const int* __restrict__ tables, int table_stride, const float* __restrict__ cos_t,
                       const float* __restrict__ sin_t, int table_rows, int rot, int pairs,
                       const float* __restrict__ q_norm, const float* __restrict__ k_norm, int v_norm, float eps,
                       TP* __restrict__ kpool, TP* __restrict__ vpool, int n_blocks, int bs, int nh, int nkv, int d, int dv,
                       int v_split, int dv_src, int whole, float qt_coef, int qt_every, int* err) {
  __shared__ float red[2][8];
  pdl_trigger();
  pdl_wait();
  const int row = blockIdx.x;
  const int seq = seq_of_row[row];
  if (seq < 0) return;
  const int pos = positions[row];
  const int half = rot / 2;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, n_warps = blockDim.x >> 5;
  T* base = qkv + (size_t)row * ld;
  float inv_whole[2] = {1.f, 1.f};  // of q and of k, when the norm is over the whole projection
  if (whole) {
    float sq = 0.f, sk = 0.f;
    for (int i = threadIdx.x; i < nh * d; i += blockDim.x) { const float v = to_f32(base[i]); sq = fmaf(v, v, sq); }
    for (int i = threadIdx.x; i < nkv * d; i += blockDim.x) { const float v = to_f32(base[k_col + i]); sk = fmaf(v, v, sk); }
    sq = warp_sum(sq);
    sk = warp_sum(sk);
    if (lane == 0) { red[0][warp] = sq; red[1][warp] = sk; }
    __syncthreads();  // (also: every value is read before any thread rewrites q in place)
    float tq = 0.f, tk = 0.f;
    for (int i = 0; i < n_warps; ++i) { tq += red[0][i]; tk += red[1][i]; }
    inv_whole[0] = 1.f / sqrtf(tq / (float)(nh * d) + eps);
    if (nkv > 0) inv_whole[1] = 1.f / sqrtf(tk / (float)(nkv * d) + eps);
  }
  const float q_mul = (qt_every > 0 && pos >= 0) ? 1.f + qt_coef * logf((float)((pos + 1) / qt_every + 1)) : 1.f;
  long long page_row = -1;
  if (nkv > 0) {
    int blk = pos >= 0 ? tables[(size_t)seq * table_stride + pos / bs] : -1;
    if (blk < 0 || blk >= n_blocks) {
      if (threadIdx.x == 0 && err) atomicExch(err, CUCA_ERR_BLOCK_RANGE);
    } else {
      page_row = (long long)blk * nkv * bs + (pos % bs);
    }
  }
  const bool in_table = pos >= 0 && pos < table_rows;
  if (!in_table && half > 0 && threadIdx.x == 0 && err) atomicExch(err, CUCA_ERR_TOKEN_RANGE);
  const float* cr = cos_t + (size_t)(in_table ? pos : 0) * half;
  const float* sr = sin_t + (size_t)(in_table ? pos : 0) * half;
  const long long slab_rows = (long long)n_blocks * nkv * bs;
  for (int head = warp; head < nh + 2 * nkv; head += n_warps) {
    const int kind = head < nh ? 0 : (head < nh + nkv ? 1 : 2);  // q, k, v
    if (kind != 0 && page_row < 0) continue;
    const int hh = kind == 0 ? head : (kind == 1 ? head - nh : head - nh - nkv);
    const int n = kind == 2 ? dv_src : d;
    const T* src = base + (kind == 0 ? 0 : (kind == 1 ? k_col : v_col)) + (size_t)hh * n;
    const float* w = kind == 0 ? q_norm : (kind == 1 ? k_norm : nullptr);
    if (whole && w) w += (size_t)hh * d;  // the weight covers the whole projection
    const bool normed = kind == 2 ? v_norm != 0 : (w != nullptr && !whole);
    float inv = (whole && kind != 2) ? inv_whole[kind] : 1.f;
    const float mul = kind == 0 ? q_mul : 1.f;
    if (normed) {
      float ss = 0.f;
      for (int i = lane; i < n; i += 32) { const float v = to_f32(src[i]); ss = fmaf(v, v, ss); }
      inv = 1.f / sqrtf(warp_sum(ss) / (float)n + eps);
    }
    __syncwarp();  // every lane has read the head before any lane rewrites it
    if (kind == 2) {
      const int ds = dv / v_split;
      for (int e = lane; e < dv; e += 32)
        vpool[((e / ds) * slab_rows + page_row + (long long)hh * bs) * ds + e % ds] =
            from_f32<TP>(e < dv_src ? to_f32(src[e]) * inv : 0.f);
      continue;
    }
    TP* dst_p = kind == 1 ? kpool + (page_row + (long long)hh * bs) * d
                          : (q_out ? q_out + ((size_t)row * nh + hh) * d : nullptr);
    T* dst_t = base + (size_t)hh * d;  // q in place
    auto put = [&](int e, float v) {
      if (dst_p) dst_p[e] = from_f32<TP>(v);
      else dst_t[e] = from_f32<T>(v);
    };
    for (int i = lane; i < half + (d - rot); i += 32) {
      if (i < half) {
        const int ia = pairs ? 2 * i : i, ib = pairs ? 2 * i + 1 : i + half;
        const float c = in_table ? cr[i] : 1.f, sn = in_table ? sr[i] : 0.f;
        const float a = to_f32(src[ia]) * inv * (w ? w[ia] : 1.f), b = to_f32(src[ib]) * inv * (w ? w[ib] : 1.f);
        put(ia, (a * c - b * sn) * mul);
        put(ib, (b * c + a * sn) * mul);
      } else {
        const int e = rot + (i - half);
        put(e, to_f32(src[e]) * inv * (w ? w[e] : 1.f) * mul);
      }
    }
  }
}
}  // namespace

// dtype: of the rows; pool_dtype: of the pools and of q_out (null: q in place, in the rows' type).
// whole, qt_coef, qt_every: see the kernel (0, 0, 0: norms per head, no query temperature).
CUCA_API int cuca_norm_rope_store_w(void* qkv, int dtype, int ld, int k_col, int v_col, void* q_out, int pool_dtype,
                                    const int* positions, const int* seq_of_row, const int* tables, int table_stride,
                                    const float* cos_t, const float* sin_t, int table_rows, int rot, int pairs,
                                    const float* q_norm, const float* k_norm, int v_norm, float eps, void* kpool,
                                    void* vpool, int n_blocks, int bs, int n_rows, int nh, int nkv, int d, int dv,
                                    int v_split, int dv_src, int whole, float qt_coef, int qt_every, int* err,
                                    cudaStream_t stream) {
  if (n_rows == 0) return 0;
  CUCA_REQUIRE(!whole || (q_norm && (nkv == 0 || k_norm) && !v_norm),
               "norm_rope_store: a norm over the whole projection needs both weights and takes no value norm");
  if (dv_src <= 0) dv_src = dv;
  CUCA_REQUIRE(dv_src <= dv, "norm_rope_store: rows with %d values a head do not fit a pool of %d", dv_src, dv);
  CUCA_REQUIRE(rot >= 0 && rot <= d && rot % 2 == 0, "norm_rope_store: rotary size %d does not fit head size %d", rot, d);
  CUCA_REQUIRE(bs > 0 && nh > 0 && nkv >= 0 && d > 0 && dv > 0, "norm_rope_store: bad sizes");
  CUCA_REQUIRE(v_split >= 1 && dv % v_split == 0, "norm_rope_store: %d slabs do not divide value size %d", v_split, dv);
#define NRS(T, TP)                                                                                                    \
  cuca_launch(norm_rope_store_kernel<T, TP>, dim3(n_rows), dim3(256), 0, stream, true, (T*)qkv, ld, k_col, v_col,      \
              (TP*)q_out, positions, seq_of_row, tables, table_stride, cos_t, sin_t, table_rows, rot, pairs, q_norm,   \
              k_norm, v_norm, eps, (TP*)kpool, (TP*)vpool, n_blocks, bs, nh, nkv, d, dv, v_split, dv_src, whole,       \
              qt_coef, qt_every, err)
  if (dtype == CUCA_F32 && pool_dtype == CUCA_F32) NRS(float, float);
  else if (dtype == CUCA_BF16 && pool_dtype == CUCA_BF16) NRS(__nv_bfloat16, __nv_bfloat16);
  else if (dtype == CUCA_F32 && pool_dtype == CUCA_BF16) {
    CUCA_REQUIRE(q_out != nullptr, "norm_rope_store: 32-bit rows with 16-bit pools need a place for q");
    NRS(float, __nv_bfloat16);
  } else CUCA_REQUIRE(false, "norm_rope_store: unsupported dtypes %d/%d", dtype, pool_dtype);
#undef NRS
  CUCA_CHECK_LAUNCH("norm_rope_store");
  return 0;
}

CUCA_API int cuca_norm_rope_store(void* qkv, int dtype, int ld, int k_col, int v_col, void* q_out, int pool_dtype,
                                  const int* positions, const int* seq_of_row, const int* tables, int table_stride,
                                  const float* cos_t, const float* sin_t, int table_rows, int rot, int pairs,
                                  const float* q_norm, const float* k_norm, int v_norm, float eps, void* kpool,
                                  void* vpool, int n_blocks, int bs, int n_rows, int nh, int nkv, int d, int dv,
                                  int v_split, int dv_src, int* err, cudaStream_t stream) {
  return cuca_norm_rope_store_w(qkv, dtype, ld, k_col, v_col, q_out, pool_dtype, positions, seq_of_row, tables,
                                table_stride, cos_t, sin_t, table_rows, rot, pairs, q_norm, k_norm, v_norm, eps, kpool,
                                vpool, n_blocks, bs, n_rows, nh, nkv, d, dv, v_split, dv_src, 0, 0.f, 0, err, stream);
}
