// Row normalisation (layernorm, groupnorm, rms-norm) with centred two-pass statistics:
//   mean = sum(x)/L, var = sum((x-mean)^2)/L, rstd = 1/sqrt(var + eps),
//   y = (x-mean)*rstd * w[widx] + b[widx]      (rms-norm: the same with mean fixed at 0,
//   the chain of pipeline/tilelang/core.py:735-776),
// the arithmetic of the reference's primitive-op chains (pipeline/tilelang/core.py:1334-1374
// for layernorm, :187-232 for groupnorm) as verify/interpreter.py executes them.  The
// reference's own CUDA layernorm (kernels/layernorm.cuh) uses E[x^2]-mean^2; the centred
// form is kept here because the metamorphic shift relations punish the one-pass form.
//
// A "row" is L contiguous elements.  For layernorm L = N and widx = column; for groupnorm
// over X[N,C,HW] a row is one (sample, group) = (C/G)*HW contiguous elements and
// widx = channel = (linear index / HW) % C.  Both are the mapping
//   widx = (linear / affine_inner) % affine_period.
//
// HBM-bound: the row is read once with 128-bit loads and stays in registers for both
// statistics passes and the normalisation; x is never re-read from memory.
//   L <= 1024   : one warp per row;
//   L <= 16384  : one CTA per row (256..1024 threads);
//   L <= 131072 : one thread-block cluster of 2..8 CTAs (256..1024 threads) per row, partial
//                 sums exchanged through distributed shared memory;
//   larger      : one CTA per row streaming the row three times (passes 2 and 3 hit L2).
#include <cooperative_groups.h>

#include <cstdlib>
#include <map>
#include <mutex>
#include <tuple>

#include "async.cuh"
#include <type_traits>

#include "common.cuh"
#include "rowio.cuh"

// Cache-streaming loads and stores for the rows of the register-resident kernels.  Measured on f32 [8192,4096], same GPU,
// libraries loaded in turn: both on, layernorm 45.3 -> 44.4 us and rms-norm 45.1 -> 43.6 us; loads alone 46.9 / 45.5 us
// (worse), stores alone no change; the residual form loses with either (63.5 -> 66.3 us with streaming loads), and so
// does softmax (23.1 -> 24.0 us with both), which therefore keeps ordinary loads and stores.
#ifndef NORM_LD
#define NORM_LD true
#define NORM_ST true
#define NORM_RES_LD false
#define NORM_RES_ST false
#endif

namespace cg = cooperative_groups;

namespace ib200 {
namespace {

enum Affine { AFF_NONE = 0, AFF_COL = 1, AFF_GENERIC = 2 };

struct AffineMap {  // widx = (linear / inner) % period, evaluated without 64-bit division per element
  FastDiv inner, period;
  int nowrap;  // rows start on a multiple of `inner` and never run past `period`: no modulo per element
  int small;   // rows*cols < 2^31: the row origin needs no 64-bit division
  int centre;  // 1: subtract the row mean (layernorm / groupnorm); 0: rms-norm, y = x * rsqrt(mean(x^2) + eps)
  int act;     // a ReLU inside the normalisation: 1 on the normalised value before the affine map, 2 on the result after it
  // residual form (f32, rows up to 16384 elements): the normalised value is x + res (+ rbias[col]), summed as
  // the rows are loaded, in that order, so that the sum never makes a round trip through HBM
  const void* res;
  const void* rbias;
};

// v <- v + res_row (+ bias); padding columns stay 0
template <typename T, typename TW, int NV, bool VEC>
__device__ __forceinline__ void add_residual(float (&v)[NV][4], const T* __restrict__ res_row, const TW* __restrict__ bias, int cols, int tid,
                                             int nthreads) {
  float t[NV][4];
  load_row<T, NV, VEC, NORM_RES_LD>(res_row, cols, tid, nthreads, 0.0f, t);
#pragma unroll
  for (int i = 0; i < NV; ++i)
#pragma unroll
    for (int k = 0; k < 4; ++k) v[i][k] += t[i][k];
  if (bias) {
    load_row<TW, NV, VEC>(bias, cols, tid, nthreads, 0.0f, t);
#pragma unroll
    for (int i = 0; i < NV; ++i)
#pragma unroll
      for (int k = 0; k < 4; ++k) v[i][k] += t[i][k];
  }
}

template <int NV> __device__ __forceinline__ float local_sum(const float (&v)[NV][4]) {
  float s = 0.0f;
#pragma unroll
  for (int i = 0; i < NV; ++i) s += (v[i][0] + v[i][1]) + (v[i][2] + v[i][3]);
  return s;
}

// v <- v - mean on valid columns (0 on padding); returns the local sum of squares.
template <int NV, bool VEC>
__device__ __forceinline__ float centre_and_square(float (&v)[NV][4], float mean, int cols, int tid, int nthreads) {
  float q = 0.0f;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int c = 4 * (i * nthreads + tid);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const bool valid = VEC ? (c < cols) : (c + k < cols);
      v[i][k] = valid ? v[i][k] - mean : 0.0f;
      q += v[i][k] * v[i][k];
    }
  }
  return q;
}

// groupnorm with large spatial extents: a thread block's whole segment [col_offset, col_offset +
// cols) usually lies inside one channel; then w and b are two scalars per row, which can be
// fetched before the reductions so that their latency is hidden
struct UniformAffine {
  bool valid = false;
  float w = 1.0f, b = 0.0f;
};
template <typename TW, int AFF>
__device__ __forceinline__ UniformAffine uniform_affine(const TW* __restrict__ w, const TW* __restrict__ b, int cols, int col_offset,
                                                        const AffineMap& map, uint32_t lin_q, uint32_t lin_r) {
  UniformAffine u;
  if (AFF == AFF_GENERIC && cols > 0) {
    const uint32_t first = map.inner.div(lin_r + col_offset), last = map.inner.div(lin_r + col_offset + cols - 1);
    if (first == last) {
      u.valid = true;
      uint32_t qq, idx = lin_q + first;
      if (!map.nowrap) map.period.divmod(lin_q + first, qq, idx);
      if (w) u.w = to_f32<TW>(w[idx]);
      if (b) u.b = to_f32<TW>(b[idx]);
    }
  }
  return u;
}

// v <- v*rstd*w + b.  `col0` is the column of this thread's first element of the row segment,
// `lin_q` / `lin_r` are quotient and remainder of the row's first linear index by affine_inner.
template <typename TW, int NV, bool VEC, int AFF>
__device__ __forceinline__ void normalise(float (&v)[NV][4], float rstd, const TW* __restrict__ w, const TW* __restrict__ b,
                                          int cols, int col_offset, int tid, int nthreads, const AffineMap& map,
                                          uint32_t lin_q, uint32_t lin_r, const UniformAffine& uni) {
  const bool uniform = uni.valid;
  const float w_uni = uni.w, b_uni = uni.b;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int c = 4 * (i * nthreads + tid);
    if (VEC && c >= cols) continue;
    float wv[4] = {1.f, 1.f, 1.f, 1.f}, bv[4] = {0.f, 0.f, 0.f, 0.f};
    if (AFF == AFF_COL) {
      if (VEC) {
        if (w) load4<TW>(w + col_offset + c, wv);
        if (b) load4<TW>(b + col_offset + c, bv);
      } else {
#pragma unroll
        for (int k = 0; k < 4; ++k)
          if (c + k < cols) {
            if (w) wv[k] = to_f32<TW>(w[col_offset + c + k]);
            if (b) bv[k] = to_f32<TW>(b[col_offset + c + k]);
          }
      }
    } else if (AFF == AFF_GENERIC) {
      if (uniform) {  // the whole segment lies in one channel: scalars fetched once, above
#pragma unroll
        for (int k = 0; k < 4; ++k) { wv[k] = w_uni; bv[k] = b_uni; }
      } else if (VEC && (map.inner.d & 3u) == 0) {  // the 4 elements share one channel
        const uint32_t ch = map.period.d == 1 ? 0u : (lin_q + map.inner.div(lin_r + col_offset + c));
        uint32_t qq, idx = ch;
        if (!map.nowrap) map.period.divmod(ch, qq, idx);
        const float ws = w ? to_f32<TW>(w[idx]) : 1.f, bs = b ? to_f32<TW>(b[idx]) : 0.f;
#pragma unroll
        for (int k = 0; k < 4; ++k) { wv[k] = ws; bv[k] = bs; }
      } else {
#pragma unroll
        for (int k = 0; k < 4; ++k)
          if (c + k < cols) {
            uint32_t qq, idx;
            map.period.divmod(lin_q + map.inner.div(lin_r + col_offset + c + k), qq, idx);
            if (w) wv[k] = to_f32<TW>(w[idx]);
            if (b) bv[k] = to_f32<TW>(b[idx]);
          }
      }
    }
    if (map.act == 0) {
#pragma unroll
      for (int k = 0; k < 4; ++k) v[i][k] = v[i][k] * rstd * wv[k] + bv[k];
    } else {  // graphs with an activation between the statistics and the store (uniform branch: the code is the plan's)
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        float t = v[i][k] * rstd;
        if (map.act == 1) t = max_nan(t, 0.0f);
        t = t * wv[k] + bv[k];
        if (map.act == 2) t = max_nan(t, 0.0f);
        v[i][k] = t;
      }
    }
  }
}

// quotient (mod period) and remainder of a row's first linear index by affine_inner
__device__ __forceinline__ void row_origin(int64_t row, int64_t cols, const AffineMap& map, uint32_t& q, uint32_t& r) {
  if (map.small) {  // multiply-shift division: a 64-bit division here would cost more than the row's arithmetic
    const uint32_t lin = (uint32_t)row * (uint32_t)cols;
    uint32_t qq, dummy;
    map.inner.divmod(lin, qq, r);
    map.period.divmod(qq, dummy, q);
    return;
  }
  const uint64_t lin = (uint64_t)row * (uint64_t)cols;
  const uint64_t qq = lin / map.inner.d;
  r = (uint32_t)(lin - qq * map.inner.d);
  q = (uint32_t)(qq % map.period.d);
}

// all-reduce over aligned groups of LANES lanes (the whole warp takes part in every shuffle)
template <int LANES> __device__ __forceinline__ float lanes_sum(float v) {
#pragma unroll
  for (int o = LANES / 2; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// LANES lanes per row: 32 for rows of 65..1024 elements, 16 or 8 for shorter ones, so that a warp
// works on 2 or 4 rows at a time and no lane holds only padding (layernorm [1048576,64] ran at 0.42
// of HBM peak with a whole warp per row).
template <typename T, typename TW, int NV, bool VEC, int AFF, bool RES, int LANES>
__global__ void __launch_bounds__(128) norm_warp(const T* __restrict__ x, const TW* __restrict__ w, const TW* __restrict__ b,
                                                 T* __restrict__ y, float* __restrict__ mean_out, float* __restrict__ rstd_out,
                                                 int64_t rows, int cols, float eps, AffineMap map) {
  constexpr int kRowsPerWarp = 32 / LANES;
  const int lane = (threadIdx.x & 31) % LANES, which = (threadIdx.x & 31) / LANES;
  const int64_t stride = (int64_t)gridDim.x * (blockDim.x >> 5) * kRowsPerWarp;
  // the loop bound is the same for every lane of a warp: the shuffles need all of them
  for (int64_t r0 = ((int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5)) * kRowsPerWarp; r0 < rows; r0 += stride) {
    const bool live = r0 + which < rows;
    const int64_t r = live ? r0 + which : rows - 1;  // lanes past the last row recompute it and store nothing
    float v[NV][4];
    load_row<T, NV, VEC, (RES ? NORM_RES_LD : NORM_LD)>(x + r * cols, cols, lane, LANES, 0.0f, v);
    if (RES) add_residual<T, TW, NV, VEC>(v, static_cast<const T*>(map.res) + r * cols, static_cast<const TW*>(map.rbias), cols, lane, LANES);
    const float mean = map.centre ? lanes_sum<LANES>(local_sum<NV>(v)) / (float)cols : 0.0f;
    const float var = lanes_sum<LANES>(centre_and_square<NV, VEC>(v, mean, cols, lane, LANES)) / (float)cols;
    const float rstd = 1.0f / sqrtf(var + eps);
    uint32_t lq = 0, lr = 0;
    if (AFF == AFF_GENERIC) row_origin(r, cols, map, lq, lr);
    normalise<TW, NV, VEC, AFF>(v, rstd, w, b, cols, 0, lane, LANES, map, lq, lr, uniform_affine<TW, AFF>(w, b, cols, 0, map, lq, lr));
    if (live) {
      store_row<T, NV, VEC, (RES ? NORM_RES_ST : NORM_ST)>(y + r * cols, cols, lane, LANES, v);
      if (lane == 0) {
        if (mean_out) mean_out[r] = mean;
        if (rstd_out) rstd_out[r] = rstd;
      }
    }
  }
}

// Mean and sum of squared deviations of a row whose every thread holds exactly NV*4 values, with ONE block barrier:
// each thread takes the moments of its own values about their own mean (exact two-pass on 4*NV numbers), and equal-sized
// sets merge without a division -- mean = (ma + mb) / 2, M2 = M2a + M2b + (mb - ma)^2 * n / 2 (Chan, Golub, LeVeque for
// na = nb = n) -- through a shuffle butterfly inside the warp and another over the warps' results.  Same arithmetic class
// as the centred two-pass form (no sum of raw squares anywhere), one barrier and ten shuffles fewer per row.
template <int NV, int THREADS>
__device__ __forceinline__ void block_moments_full(const float (&v)[NV][4], float (*slots)[2], float& mean, float& m2) {
  constexpr float kOwn = (float)(NV * 4);
  float mu = local_sum<NV>(v) * (1.0f / kOwn), q = 0.0f;
#pragma unroll
  for (int i = 0; i < NV; ++i)
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float d = v[i][k] - mu;
      q = fmaf(d, d, q);
    }
  float half = kOwn * 0.5f;  // n / 2 of the sets being merged
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const float mo = __shfl_xor_sync(0xffffffffu, mu, o), qo = __shfl_xor_sync(0xffffffffu, q, o);
    const float d = mo - mu;
    q = (q + qo) + d * d * half;
    mu = 0.5f * (mu + mo);
    half *= 2.0f;
  }
  constexpr int kWarps = THREADS / 32;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) { slots[warp][0] = mu; slots[warp][1] = q; }
  __syncthreads();
  mu = slots[lane & (kWarps - 1)][0];
  q = slots[lane & (kWarps - 1)][1];
#pragma unroll
  for (int o = 1; o < kWarps; o <<= 1) {  // lanes 0 .. kWarps-1 hold the warps' results; the other lanes mirror them
    const float mo = __shfl_xor_sync(0xffffffffu, mu, o), qo = __shfl_xor_sync(0xffffffffu, q, o);
    const float d = mo - mu;
    q = (q + qo) + d * d * half;
    mu = 0.5f * (mu + mo);
    half *= 2.0f;
  }
  mean = mu;
  m2 = q;
}

// 256-thread CTAs are held to 51 registers so that five are resident per SM (measured on f32 [8192,4096]:
// layernorm 0.80 -> 0.86 of HBM peak, rms-norm 0.86 -> 0.90; six CTAs spill and gain nothing); with 8 values
// per thread (rows of 1025..2048 elements) all eight fit: [32768,2048] 0.78 -> 0.90
template <typename T, typename TW, int THREADS, int NV, bool VEC, int AFF, bool RES>
__global__ void __launch_bounds__(THREADS, THREADS == 256 ? (NV <= 2 ? 8 : 5) : 1) norm_block(const T* __restrict__ x, const TW* __restrict__ w,
                                                      const TW* __restrict__ b, T* __restrict__ y,
                                                      float* __restrict__ mean_out, float* __restrict__ rstd_out,
                                                      int64_t rows, int cols, float eps, AffineMap map) {
  __shared__ float slots[2][32];
  __shared__ float mslots[2][THREADS / 32][2];
  int parity = 0;
  const bool full = map.centre && cols == NV * 4 * THREADS;  // every thread holds NV*4 values of the row
  for (int64_t r = blockIdx.x; r < rows; r += gridDim.x, parity ^= 1) {
    float v[NV][4];
    load_row<T, NV, VEC, (RES ? NORM_RES_LD : NORM_LD)>(x + r * cols, cols, threadIdx.x, THREADS, 0.0f, v);
    if (RES) add_residual<T, TW, NV, VEC>(v, static_cast<const T*>(map.res) + r * cols, static_cast<const TW*>(map.rbias), cols, threadIdx.x, THREADS);
    float mean, var;
    if (full) {  // one barrier per row (slots alternate by row parity)
      float m2;
      block_moments_full<NV, THREADS>(v, mslots[parity], mean, m2);
      var = m2 / (float)cols;
#pragma unroll
      for (int i = 0; i < NV; ++i)
#pragma unroll
        for (int k = 0; k < 4; ++k) v[i][k] -= mean;
    } else {
      // two reductions per centred row alternate between the two slot arrays; the single reduction of an
      // uncentred (rms) row alternates by row parity, so that a fast warp never overwrites partials a slow one still reads
      mean = map.centre ? block_reduce<SumOp>(local_sum<NV>(v), slots[0]) / (float)cols : 0.0f;
      var = block_reduce<SumOp>(centre_and_square<NV, VEC>(v, mean, cols, threadIdx.x, THREADS), slots[map.centre ? 1 : parity]) / (float)cols;
    }
    const float rstd = 1.0f / sqrtf(var + eps);
    uint32_t lq = 0, lr = 0;
    if (AFF == AFF_GENERIC) row_origin(r, cols, map, lq, lr);
    normalise<TW, NV, VEC, AFF>(v, rstd, w, b, cols, 0, threadIdx.x, THREADS, map, lq, lr, uniform_affine<TW, AFF>(w, b, cols, 0, map, lq, lr));
    store_row<T, NV, VEC, (RES ? NORM_RES_ST : NORM_ST)>(y + r * cols, cols, threadIdx.x, THREADS, v);
    if (threadIdx.x == 0) {
      if (mean_out) mean_out[r] = mean;
      if (rstd_out) rstd_out[r] = rstd;
    }
  }
}

// One cluster of `csize` CTAs per row: CTA k keeps columns [k*seg, (k+1)*seg) in registers and
// computes the statistics of its own segment exactly (sum -> segment mean -> centred sum of
// squares, two block reductions).  The segments are then merged with the pairwise update
//   mean = sum_k n_k*mean_k / L,   M2 = sum_k M2_k + sum_k n_k*(mean_k - mean)^2,
// which is algebraically the centred two-pass variance of the whole row.  Each CTA pushes its
// (mean_k, M2_k, n_k) into every peer's shared memory, so there is a single cluster barrier
// per row and afterwards every CTA reads only its own shared memory (no CTA can be exited
// while a peer still needs it).  The barrier arrive issued at kernel entry and waited on before
// the first remote store guarantees that every CTA of the cluster has started.
__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }

template <typename T, typename TW, int THREADS, int NV, bool VEC, int AFF>
__global__ void __launch_bounds__(THREADS) norm_cluster(const T* __restrict__ x, const TW* __restrict__ w,
                                                        const TW* __restrict__ b, T* __restrict__ y,
                                                        float* __restrict__ mean_out, float* __restrict__ rstd_out,
                                                        int64_t rows, int cols, int seg, float eps, AffineMap map) {
  __shared__ float slots[2][32];
  __shared__ float part[8][3];  // per peer: segment mean, centred sum of squares, element count
  cg::cluster_group cluster = cg::this_cluster();
  cluster_arrive();
  const int csize = (int)cluster.num_blocks(), rank = (int)cluster.block_rank();
  const int64_t r = blockIdx.x / csize;  // grid is exactly rows * csize, so r < rows
  const int col0 = rank * seg;
  const int mine = min(seg, cols - col0) > 0 ? min(seg, cols - col0) : 0;
  float v[NV][4];
  load_row<T, NV, VEC>(x + r * cols + col0, mine, threadIdx.x, THREADS, 0.0f, v);

  const float s = block_reduce<SumOp>(local_sum<NV>(v), slots[0]);
  const float mean_k = mine > 0 && map.centre ? s / (float)mine : 0.0f;
  const float q = block_reduce<SumOp>(centre_and_square<NV, VEC>(v, mean_k, mine, threadIdx.x, THREADS), slots[1]);

  cluster_wait();  // every CTA of the cluster is running: remote shared memory may be written
  if (threadIdx.x < csize) {
    float* dst = cluster.map_shared_rank(&part[rank][0], threadIdx.x);
    dst[0] = mean_k;
    dst[1] = q;
    dst[2] = (float)mine;
  }
  cluster_arrive();
  cluster_wait();

  float mean = 0.0f;
  for (int k = 0; k < csize; ++k) mean += part[k][2] * part[k][0];
  mean /= (float)cols;
  float m2 = 0.0f;
  for (int k = 0; k < csize; ++k) {
    const float d = part[k][0] - mean;
    m2 += part[k][1] + part[k][2] * d * d;
  }
  const float rstd = 1.0f / sqrtf(m2 / (float)cols + eps);
  const float shift = mean_k - mean;  // registers hold x - mean_k
#pragma unroll
  for (int i = 0; i < NV; ++i)
#pragma unroll
    for (int k = 0; k < 4; ++k) v[i][k] += shift;

  uint32_t lq = 0, lr = 0;
  if (AFF == AFF_GENERIC) row_origin(r, cols, map, lq, lr);
  normalise<TW, NV, VEC, AFF>(v, rstd, w, b, mine, col0, threadIdx.x, THREADS, map, lq, lr,
                              uniform_affine<TW, AFF>(w, b, mine, col0, map, lq, lr));
  store_row<T, NV, VEC>(y + r * cols + col0, mine, threadIdx.x, THREADS, v);
  if (rank == 0 && threadIdx.x == 0) {
    if (mean_out) mean_out[r] = mean;
    if (rstd_out) rstd_out[r] = rstd;
  }
}

// Persistent, software-pipelined variant for rows of up to 8 x 4096 elements: a group of
// `csize` CTAs (a thread-block cluster when csize > 1) owns rows group, group + n_groups, ...
// Each CTA stages its segment of a row into shared memory with one bulk asynchronous copy (TMA,
// completion on an mbarrier).  Two stages: as soon as a row has been read into registers its stage
// is refilled with the row after next, so two rows are on their way while one is worked on.
// What bounds this kernel is the chain of waits inside a row, not the copies, so the chain is as
// short as it gets: every thread watches the data barrier itself, the statistics are taken in ONE
// pass (sums of x - pivot and of its square, pivot = mean of the segment's first four elements) with
// ONE block barrier, they travel between the CTAs as asynchronous shared-memory stores that count
// bytes on the receiver's mbarrier (no cluster-wide barrier, no fence on the row stores in
// flight), and every warp merges the peers' statistics on its own.  Two sets of exchange slots: a
// peer can run at most one row ahead.  Measured on groupnorm f32 [32,256,4096] with 32 groups:
// 57.6 us with a two-pass form that needed four block barriers per row, 53.0 us in this form.
template <typename T, typename TW, int AFF, bool CLUSTER, int NV>
__global__ void __launch_bounds__(256) norm_pipe(const T* __restrict__ x, const TW* __restrict__ w, const TW* __restrict__ b,
                                                 T* __restrict__ y, float* __restrict__ mean_out, float* __restrict__ rstd_out,
                                                 int64_t rows, int cols, int seg, int stage_bytes, float eps, AffineMap map,
                                                 int32_t* status) {
  constexpr int THREADS = 256;
  extern __shared__ __align__(128) unsigned char stage_mem[];
  __shared__ uint64_t bar[2];   // staged row segments
  __shared__ uint64_t xbar[2];  // statistics received from the peers
  __shared__ float slots[2][16];  // [row parity][s1 of warps 0..7, s2 of warps 0..7]
  __shared__ float part[2][8][3];
  int csize = 1, rank = 0;
  if (CLUSTER) {
    cg::cluster_group cluster = cg::this_cluster();
    csize = (int)cluster.num_blocks();
    rank = (int)cluster.block_rank();
  }
  const int64_t n_groups = gridDim.x / csize, group = blockIdx.x / csize;
  const int col0 = rank * seg;
  const int mine = min(seg, cols - col0) > 0 ? min(seg, cols - col0) : 0;
  const uint32_t bytes = (uint32_t)mine * sizeof(T);
  if (threadIdx.x == 0) {
    mbarrier_init(&bar[0], 1);
    mbarrier_init(&bar[1], 1);
    mbarrier_init(&xbar[0], 1);
    mbarrier_init(&xbar[1], 1);
    mbarrier_init_fence();
  }
  __syncthreads();
  if (CLUSTER) cluster_arrive();
  if (threadIdx.x == 0 && bytes) {  // the first two rows of this group are requested at once
    for (int k = 0; k < 2; ++k)
      if (group + k * n_groups < rows) {
        mbarrier_expect_tx(&bar[k], bytes);
        bulk_load(stage_mem + k * stage_bytes, x + (group + k * n_groups) * cols + col0, bytes, &bar[k]);
      }
  }
  int it = 0;
  for (int64_t r = group; r < rows; r += n_groups, ++it) {
    const int st = it & 1;
    uint32_t lq = 0, lr = 0;
    if (AFF == AFF_GENERIC) row_origin(r, cols, map, lq, lr);
    const UniformAffine uni = uniform_affine<TW, AFF>(w, b, mine, col0, map, lq, lr);  // in flight during the reductions
    // every thread watches the mbarrier itself (the wait suspends in hardware): no block barrier between the
    // arrival of the data and the arithmetic
    if (bytes && !mbarrier_wait_bounded(&bar[st], (it >> 1) & 1) && status) atomicCAS(status, 0, 5);
    const T* staged = reinterpret_cast<const T*>(stage_mem + st * stage_bytes);
    float v[NV][4];
    load_row<T, NV, true>(staged, mine, threadIdx.x, THREADS, 0.0f, v);

    // One pass, one block reduction: sums of d = x - pivot and of d*d, the pivot being the mean of the segment's
    // first four elements (a sample of the row keeps s2 - s1*s1/n far from cancellation; rms rows use pivot 0,
    // where s2 is the wanted sum itself).  v keeps d; the final centring is one more add, below.
    float pivot = 0.0f;
    if (map.centre && mine >= 4) {
      float h[4];
      load4<T>(staged, h);
      pivot = ((h[0] + h[1]) + (h[2] + h[3])) * 0.25f;
    }
    float s1 = 0.0f, s2 = 0.0f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const bool valid = 4 * (i * THREADS + (int)threadIdx.x) < mine;
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float d = valid ? v[i][k] - pivot : 0.0f;
        v[i][k] = d;
        s1 += d;
        s2 = fmaf(d, d, s2);
      }
    }
    {
      s1 = warp_reduce<SumOp>(s1);
      s2 = warp_reduce<SumOp>(s2);
      const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
      if (lane == 0) { slots[st][warp] = s1; slots[st][8 + warp] = s2; }
      __syncthreads();  // the only block barrier of the row
      // the row now lives in registers: its stage is refilled at once with the row after next, so that two
      // rows are on their way while this one is merged, normalised and stored
      if (threadIdx.x == 0 && bytes && r + 2 * n_groups < rows) {
        mbarrier_expect_tx(&bar[st], bytes);
        bulk_load(stage_mem + st * stage_bytes, x + (r + 2 * n_groups) * cols + col0, bytes, &bar[st]);
      }
      const float t = lane < 16 ? slots[st][lane] : 0.0f;
      s1 = lanes_sum<8>(t);                                  // lanes 0..7 hold s1, lanes 8..15 s2
      s2 = __shfl_sync(0xffffffffu, s1, 8);
      s1 = __shfl_sync(0xffffffffu, s1, 0);
    }
    const float mean_k = map.centre && mine > 0 ? pivot + s1 / (float)mine : 0.0f;
    const float q = map.centre && mine > 0 ? fmaxf(s2 - s1 * s1 / (float)mine, 0.0f) : s2;
    float mean = mean_k, m2 = q;
    if (CLUSTER) {
      if (it == 0) cluster_wait();  // all CTAs of the cluster are running and have initialised their barriers
      // every CTA sends its (mean, M2, count) to every peer with stores that count bytes on the
      // receiver's mbarrier; no cluster-wide barrier, no fence on the row stores in flight
      if (threadIdx.x == 0) mbarrier_expect_tx(&xbar[st], (uint32_t)csize * 12u);
      if (threadIdx.x < csize) {
        const uint32_t dst = cluster_map(&part[st][rank][0], threadIdx.x), rbar = cluster_map(&xbar[st], threadIdx.x);
        remote_store_signal(dst, mean_k, rbar);
        remote_store_signal(dst + 4, q, rbar);
        remote_store_signal(dst + 8, (float)mine, rbar);
      }
      // every warp waits for the peers' statistics and merges them on its own (lane k owns peer k, two
      // shuffle reductions): no second block barrier
      if (!mbarrier_wait_bounded(&xbar[st], (it >> 1) & 1) && status) atomicCAS(status, 0, 6);
      const int lane = threadIdx.x & 31;
      const bool have = lane < csize;
      const float mk = have ? part[st][lane][0] : 0.0f, qk = have ? part[st][lane][1] : 0.0f, nk = have ? part[st][lane][2] : 0.0f;
      mean = warp_reduce<SumOp>(nk * mk) / (float)cols;
      const float dk = mk - mean;
      m2 = warp_reduce<SumOp>(qk + nk * dk * dk);
    }
    {
      const float shift = pivot - mean;  // d + (pivot - mean) = x - mean
#pragma unroll
      for (int i = 0; i < NV; ++i)
#pragma unroll
        for (int k = 0; k < 4; ++k) v[i][k] += shift;
    }
    const float rstd = 1.0f / sqrtf(m2 / (float)cols + eps);
    normalise<TW, NV, true, AFF>(v, rstd, w, b, mine, col0, threadIdx.x, THREADS, map, lq, lr, uni);
    store_row<T, NV, true>(y + r * cols + col0, mine, threadIdx.x, THREADS, v);
    if (rank == 0 && threadIdx.x == 0) {
      if (mean_out) mean_out[r] = mean;
      if (rstd_out) rstd_out[r] = rstd;
    }
  }
}

template <typename T, typename TW, int AFF>
__global__ void __launch_bounds__(1024) norm_stream(const T* __restrict__ x, const TW* __restrict__ w, const TW* __restrict__ b,
                                                    T* __restrict__ y, float* __restrict__ mean_out, float* __restrict__ rstd_out,
                                                    int64_t rows, int64_t cols, float eps, int64_t inner, int64_t period, int centre, int act) {
  __shared__ float slots[2][32];
  for (int64_t r = blockIdx.x; r < rows; r += gridDim.x) {
    const T* xr = x + r * cols;
    T* yr = y + r * cols;
    float s = 0.0f;
    for (int64_t c = threadIdx.x; c < cols; c += blockDim.x) s += to_f32<T>(xr[c]);
    const float mean = centre ? block_reduce<SumOp>(s, slots[0]) / (float)cols : 0.0f;
    float q = 0.0f;
    for (int64_t c = threadIdx.x; c < cols; c += blockDim.x) {
      const float d = to_f32<T>(xr[c]) - mean;
      q += d * d;
    }
    const float rstd = 1.0f / sqrtf(block_reduce<SumOp>(q, slots[1]) / (float)cols + eps);
    for (int64_t c = threadIdx.x; c < cols; c += blockDim.x) {
      float wv = 1.0f, bv = 0.0f;
      if (AFF != AFF_NONE) {
        const int64_t idx = AFF == AFF_COL ? c : ((r * cols + c) / inner) % period;
        if (w) wv = to_f32<TW>(w[idx]);
        if (b) bv = to_f32<TW>(b[idx]);
      }
      float t = (to_f32<T>(xr[c]) - mean) * rstd;
      if (act == 1) t = max_nan(t, 0.0f);
      t = t * wv + bv;
      if (act == 2) t = max_nan(t, 0.0f);
      yr[c] = from_f32<T>(t);
    }
    if (threadIdx.x == 0) {
      if (mean_out) mean_out[r] = mean;
      if (rstd_out) rstd_out[r] = rstd;
    }
  }
}

struct Args {
  const void *x, *w, *b;
  void* y;
  float *mean, *rstd;
  int64_t rows, cols, inner, period;
  float eps;
  cudaStream_t s;
  int32_t* status;
  int centre;
  const void *res, *rbias;
  int act;
};

// how many groups of `csize` CTAs of a kernel can be resident at once (cached per kernel)
template <typename K> int resident_groups(K kernel, int csize, int smem) {
  static std::mutex mu;
  static std::map<std::tuple<const void*, int, int, int>, int> cache;
  int dev = 0;
  cudaGetDevice(&dev);
  const auto key = std::make_tuple(reinterpret_cast<const void*>(kernel), csize, smem, dev);
  std::lock_guard<std::mutex> lock(mu);
  auto it = cache.find(key);
  if (it != cache.end()) return it->second;
  int n = 0;
  if (csize > 1) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(csize * kSmCount);
    cfg.blockDim = dim3(256);
    cfg.dynamicSmemBytes = smem;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = csize;
    attr[0].val.clusterDim.y = attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (cudaOccupancyMaxActiveClusters(&n, kernel, &cfg) != cudaSuccess) { cudaGetLastError(); n = 0; }
  } else {
    int per_sm = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, 256, smem) != cudaSuccess) { cudaGetLastError(); per_sm = 0; }
    n = per_sm * kSmCount;
  }
  if (n <= 0) n = kSmCount / csize;
  cache[key] = n;
  return n;
}

template <typename T, typename TW, int AFF, bool CLUSTER, int NV> int launch_pipe(const Args& a, const AffineMap& map, int csize, int seg) {
  auto kernel = norm_pipe<T, TW, AFF, CLUSTER, NV>;
  const int stage_bytes = (int)(((size_t)seg * sizeof(T) + 127) & ~(size_t)127);
  const int smem = 2 * stage_bytes;
  const int64_t resident = resident_groups(kernel, csize, smem);
  const int64_t groups = a.rows < resident ? a.rows : resident;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(groups * csize));
  cfg.blockDim = dim3(256);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = a.s;
  cudaLaunchAttribute attr[1];
  if (CLUSTER) {
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = csize;
    attr[0].val.clusterDim.y = attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
  }
  cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, static_cast<const T*>(a.x), static_cast<const TW*>(a.w), static_cast<const TW*>(a.b),
                                     static_cast<T*>(a.y), a.mean, a.rstd, a.rows, (int)a.cols, seg, stage_bytes, a.eps, map, a.status);
  return e == cudaSuccess ? IB200_OK : cuda_fail(e, "norm pipelined launch");
}

template <typename T, typename TW, bool VEC, int AFF> int dispatch(const Args& a) {
  const T* x = static_cast<const T*>(a.x);
  T* y = static_cast<T*>(a.y);
  const TW *w = static_cast<const TW*>(a.w), *b = static_cast<const TW*>(a.b);
  constexpr bool kResidualBuilt = std::is_same<T, float>::value && std::is_same<TW, float>::value;
  if (a.res && (!kResidualBuilt || a.cols > 16384)) return fail(IB200_ERR_UNSUPPORTED, "norm: the residual form covers f32 rows of up to 16384 elements");
  AffineMap map;
  map.res = a.res;
  map.rbias = a.rbias;
  map.centre = a.centre;
  map.act = a.act;
  map.nowrap = 0;
  map.small = a.rows * a.cols < ((int64_t)1 << 31);
  if (AFF == AFF_GENERIC) {
    map.inner = FastDiv((uint32_t)a.inner);
    map.period = FastDiv((uint32_t)a.period);
    map.nowrap = a.cols % a.inner == 0 && a.period % (a.cols / a.inner) == 0;
  }
  const int c = (int)a.cols;
  if (VEC && !a.res && a.cols > 4096 && a.cols <= 32768 && (a.cols * sizeof(T)) % 16 == 0) {
#ifdef IB200_AB_KNOBS  // A/B builds only: IB200_NORM_PIPE=0 falls back to the one-shot cluster kernel
    static const bool enabled = !(std::getenv("IB200_NORM_PIPE") && std::getenv("IB200_NORM_PIPE")[0] == '0');
#else
    constexpr bool enabled = true;
#endif
    int csize = 1;
    while ((int64_t)csize * 4096 < a.cols) csize *= 2;
    int seg = (int)((a.cols + csize - 1) / csize);
    seg = (seg + 7) & ~7;  // segment starts and sizes stay multiples of 16 bytes for 2- and 4-byte elements
    if (enabled && ((size_t)seg * sizeof(T)) % 16 == 0)
      return csize == 1 ? launch_pipe<T, TW, AFF, false, 4>(a, map, 1, seg) : launch_pipe<T, TW, AFF, true, 4>(a, map, csize, seg);
  }
#define IB200_WARP(NV) IB200_WARP_L(NV, 32)
#define IB200_WARP_L(NV, LANES)                                                                                   \
  {                                                                                                               \
    const int64_t blocks = (a.rows + 4 * (32 / LANES) - 1) / (4 * (32 / LANES));                                  \
    const int grid = (int)(blocks < (int64_t)kSmCount * 32 ? blocks : (int64_t)kSmCount * 32);                    \
    if (!a.res) norm_warp<T, TW, NV, VEC, AFF, false, LANES><<<grid, 128, 0, a.s>>>(x, w, b, y, a.mean, a.rstd, a.rows, c, a.eps, map); \
    else if constexpr (kResidualBuilt) norm_warp<T, TW, NV, VEC, AFF, true, LANES><<<grid, 128, 0, a.s>>>(x, w, b, y, a.mean, a.rstd, a.rows, c, a.eps, map); \
  }
#define IB200_BLOCK(TH, NV)                                                                                       \
  {                                                                                                               \
    const int64_t cap = (int64_t)kSmCount * (2048 / TH) * 8;                                                      \
    const int grid = (int)(a.rows < cap ? a.rows : cap);                                                          \
    if (!a.res) norm_block<T, TW, TH, NV, VEC, AFF, false><<<grid, TH, 0, a.s>>>(x, w, b, y, a.mean, a.rstd, a.rows, c, a.eps, map); \
    else if constexpr (kResidualBuilt) norm_block<T, TW, TH, NV, VEC, AFF, true><<<grid, TH, 0, a.s>>>(x, w, b, y, a.mean, a.rstd, a.rows, c, a.eps, map); \
  }
  if (a.cols <= 32) IB200_WARP_L(1, 8)
  else if (a.cols <= 64) IB200_WARP_L(1, 16)
  else if (a.cols <= 128) IB200_WARP(1)
  else if (a.cols <= 256) IB200_WARP(2)
  else if (a.cols <= 512) IB200_WARP(4)
  else if (a.cols <= 1024) IB200_WARP(8)
  else if (a.cols <= 2048) IB200_BLOCK(256, 2)
  else if (a.cols <= 4096) IB200_BLOCK(256, 4)
  else if (a.cols <= 8192) IB200_BLOCK(512, 4)
  else if (a.cols <= 16384) IB200_BLOCK(1024, 4)
  else if (a.cols <= 131072 && a.rows * 8 < (int64_t)INT32_MAX) {
    // a cluster of up to 8 CTAs per row, 16 elements per thread: the smallest CTA (256, 512 or
    // 1024 threads) whose 8-CTA cluster still covers the row keeps several CTAs per SM, so
    // the loads of one cluster overlap the reductions and stores of others
    const int threads = a.cols <= 32768 ? 256 : (a.cols <= 65536 ? 512 : 1024);
    const int64_t per_cta = (int64_t)threads * 16;
    int csize = 1;
    while ((int64_t)csize * per_cta < a.cols) csize *= 2;
    int seg = (int)((a.cols + csize - 1) / csize);
    seg = (seg + 3) & ~3;  // keep every segment start aligned to a 4-element vector
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(a.rows * csize));
    cfg.blockDim = dim3(threads);
    cfg.stream = a.s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = csize;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaError_t e;
    if (threads == 256)
      e = cudaLaunchKernelEx(&cfg, norm_cluster<T, TW, 256, 4, VEC, AFF>, x, w, b, y, a.mean, a.rstd, a.rows, c, seg, a.eps, map);
    else if (threads == 512)
      e = cudaLaunchKernelEx(&cfg, norm_cluster<T, TW, 512, 4, VEC, AFF>, x, w, b, y, a.mean, a.rstd, a.rows, c, seg, a.eps, map);
    else
      e = cudaLaunchKernelEx(&cfg, norm_cluster<T, TW, 1024, 4, VEC, AFF>, x, w, b, y, a.mean, a.rstd, a.rows, c, seg, a.eps, map);
    if (e != cudaSuccess) return cuda_fail(e, "norm cluster launch");
  } else {
    if (AFF == AFF_GENERIC && (a.rows * a.cols) / a.inner >= (int64_t)1 << 62) return fail(IB200_ERR_UNSUPPORTED, "norm: extent too large");
    const int grid = (int)(a.rows < (int64_t)kSmCount * 2 ? a.rows : (int64_t)kSmCount * 2);
    norm_stream<T, TW, AFF><<<grid, 1024, 0, a.s>>>(x, w, b, y, a.mean, a.rstd, a.rows, a.cols, a.eps, a.inner, a.period, a.centre, a.act);
  }
#undef IB200_WARP
#undef IB200_WARP_L
#undef IB200_BLOCK
  return cudaPeekAtLastError() == cudaSuccess ? IB200_OK : cuda_fail(cudaGetLastError(), "norm launch");
}

template <typename T, typename TW> int pick_mode(const Args& a) {
  bool vec = aligned16(a.x) && aligned16(a.y) && a.cols % 4 == 0;
  int aff = AFF_GENERIC;
  if (!a.w && !a.b) aff = AFF_NONE;
  else if (a.inner == 1 && a.period == a.cols) aff = AFF_COL;
  if (aff == AFF_COL && vec) vec = (!a.w || aligned16(a.w)) && (!a.b || aligned16(a.b));
  // the register-resident generic mapping divides 32-bit offsets: the per-row offset
  // (remainder + column) must stay below 2^31
  if (aff == AFF_GENERIC && (a.inner >= ((int64_t)1 << 30) || a.period >= ((int64_t)1 << 30) || a.cols >= ((int64_t)1 << 30)))
    return fail(IB200_ERR_UNSUPPORTED, "norm: affine_inner / affine_period / cols must be below 2^30");
#define IB200_GO(V, A) return dispatch<T, TW, V, A>(a)
  if (vec) {
    if (aff == AFF_NONE) IB200_GO(true, AFF_NONE);
    if (aff == AFF_COL) IB200_GO(true, AFF_COL);
    IB200_GO(true, AFF_GENERIC);
  }
  if (aff == AFF_NONE) IB200_GO(false, AFF_NONE);
  if (aff == AFF_COL) IB200_GO(false, AFF_COL);
  IB200_GO(false, AFF_GENERIC);
#undef IB200_GO
}

}  // namespace

// A status word for callers of the direct entry points, which pass none: set non-zero if a
// bounded wait for a bulk copy ever ran out (read by ib200_check_status(NULL, stream)).
static __device__ int32_t g_norm_status;

int32_t* norm_default_status() {
  static std::mutex mu;
  static int32_t* addr[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  std::lock_guard<std::mutex> lock(mu);
  if (!addr[dev]) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_norm_status) != cudaSuccess) { cudaGetLastError(); return nullptr; }
    addr[dev] = static_cast<int32_t*>(p);
  }
  return addr[dev];
}

int launch_norm_rows(const void* x, const void* w, const void* b, void* y, float* mean, float* rstd, int dtype,
                     int affine_dtype, int64_t rows, int64_t cols, int64_t affine_inner, int64_t affine_period, float eps,
                     cudaStream_t s, int32_t* status, bool centre, const void* res, const void* res_bias, void* scratch, size_t scratch_bytes,
                     int act) {
  if (!status) status = norm_default_status();
  if (rows < 0 || cols < 0) return fail(IB200_ERR_INVALID, "norm: negative extent");
  if (rows == 0 || cols == 0) return IB200_OK;
  if (beyond_any_device(rows, cols)) return fail(IB200_ERR_INVALID, "norm: more than 2^40 elements");
  if (!x || !y) return fail(IB200_ERR_INVALID, "norm: null pointer");
  if ((w || b) && (affine_inner < 1 || affine_period < 1)) return fail(IB200_ERR_INVALID, "norm: affine_inner and affine_period must be >= 1");
  if (res_bias && !res) return fail(IB200_ERR_INVALID, "norm: a residual bias needs a residual");
  if (act < 0 || act > 2) return fail(IB200_ERR_INVALID, "norm: unknown activation position");
  if (scratch && !res && act == 0) {  // few, very long rows: segments over the whole GPU (longrow.cu)
    const int rc = try_norm_segmented(x, w, b, y, mean, rstd, dtype, affine_dtype, rows, cols, affine_inner, affine_period, eps, centre ? 1 : 0,
                                      scratch, scratch_bytes, s, status);
    if (rc != 1) return rc;
  }
  Args a{x, w, b, y, mean, rstd, rows, cols, affine_inner, affine_period, eps, s, status, centre ? 1 : 0, res, res_bias, act};
  const int adt = (w || b) ? affine_dtype : dtype;
  switch (dtype) {
    case IB200_F32:
      if (adt == IB200_F32) return pick_mode<float, float>(a);
      break;
    case IB200_BF16:
      if (adt == IB200_BF16) return pick_mode<__nv_bfloat16, __nv_bfloat16>(a);
      if (adt == IB200_F32) return pick_mode<__nv_bfloat16, float>(a);
      break;
    case IB200_F16:
      if (adt == IB200_F16) return pick_mode<__half, __half>(a);
      if (adt == IB200_F32) return pick_mode<__half, float>(a);
      break;
    default: break;
  }
  return fail(IB200_ERR_UNSUPPORTED, "norm: x/y must be f32, bf16 or f16; w/b the same type or f32");
}

}  // namespace ib200
