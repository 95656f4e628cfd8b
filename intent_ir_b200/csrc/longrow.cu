// Softmax and row normalisation over rows that are too long for one CTA's registers and too few
// (or too large) for one streaming CTA per row to use the GPU: [4, 1 Mi], a whole-tensor
// layernorm, a softmax over a flattened feature map.
//
// The row is cut into segments of 8 Ki .. 64 Ki elements, one CTA each, and the work is two
// launches with nothing waiting on anything:
//   pass 1  every CTA reduces its segment, in one read, to a pair of statistics — softmax:
//           (max, sum of exp(x - max)); normalisation: (mean, sum of squared deviations from
//           that mean) — and stores the pair in scratch;
//   pass 2  every CTA folds the pairs of its row (the same tree on every run, so the result
//           does not change from run to run), then writes its segment.
// x is read twice, the second time out of L2 when the tensor fits there; the one-CTA-per-row
// streaming kernels read it three times with most of the GPU idle.  The arithmetic follows
// verify/interpreter.py:501-506 (softmax) and the centred two-pass variance of the layernorm /
// groupnorm graphs (pipeline/tilelang/core.py:1334-1374): segment means and deviations are merged
// with the pairwise update of Chan et al., which is the two-pass result up to rounding.
#include <map>
#include <mutex>
#include <tuple>

#include "common.cuh"

namespace ib200 {
namespace {

constexpr int kThreads = 512;
constexpr int64_t kMinSeg = 8192, kMaxSeg = 65536;
constexpr int kMaxSegs = 4096;

__device__ __forceinline__ float fast_exp(float t) {
  float r;
  asm("ex2.approx.f32 %0, %1;" : "=f"(r) : "f"(t * 1.4426950408889634f));
  return r;
}
// exp(a - b) for running maxima a <= b: 1 when they are equal (also when both are -inf, where a - b is NaN)
__device__ __forceinline__ float rescale(float a, float b) { return a == b ? 1.0f : fast_exp(a - b); }

// The second launch of each pair is a programmatic dependent launch: it may be scheduled while the first one is
// still draining, and waits here (a hardware dependency, not a spin) until the first has completed and its
// statistics are visible.  That hides most of the gap between the two launches, which is a third of the run time
// for a tensor of a few megabytes.
__device__ __forceinline__ void wait_for_previous_launch() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void let_next_launch_start() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

struct Seg {
  int64_t row, c0, c1;
};
__device__ __forceinline__ Seg my_segment(int64_t cols, int segs, int64_t seg_len) {
  Seg g;
  g.row = blockIdx.x / segs;
  g.c0 = (int64_t)(blockIdx.x % segs) * seg_len;
  g.c1 = g.c0 + seg_len < cols ? g.c0 + seg_len : cols;
  return g;
}

enum { AFF_NONE = 0, AFF_COL = 1, AFF_GENERIC = 2 };

// ---- softmax ---------------------------------------------------------------------------------
template <typename T, bool VEC>
__global__ void __launch_bounds__(kThreads) softmax_seg_stats(const T* __restrict__ x, float2* __restrict__ part, int64_t cols, int segs,
                                                              int64_t seg_len) {
  __shared__ float slots[2][32];
  const Seg g = my_segment(cols, segs, seg_len);
  let_next_launch_start();
  const T* xr = x + g.row * cols;
  float m = -INFINITY, s = 0.0f;  // running maximum, and the sum of exp(x - m) so far
  if (VEC) {
#pragma unroll 4
    for (int64_t c = g.c0 + 4 * threadIdx.x; c < g.c1; c += 4 * kThreads) {
      float v[4];
      load4<T>(xr + c, v);
      const float mn = max_nan(m, max_nan(max_nan(v[0], v[1]), max_nan(v[2], v[3])));
      float add = 0.0f;
      if (mn != -INFINITY) add = fast_exp(v[0] - mn) + fast_exp(v[1] - mn) + fast_exp(v[2] - mn) + fast_exp(v[3] - mn);
      s = s * rescale(m, mn) + add;
      m = mn;
    }
  } else {
    for (int64_t c = g.c0 + threadIdx.x; c < g.c1; c += kThreads) {
      const float v = to_f32<T>(xr[c]);
      const float mn = max_nan(m, v);
      s = s * rescale(m, mn) + (mn != -INFINITY ? fast_exp(v - mn) : 0.0f);
      m = mn;
    }
  }
  const float big = block_reduce<MaxOp>(m, slots[0]);
  const float total = block_reduce<SumOp>(s * rescale(m, big), slots[1]);
  if (threadIdx.x == 0) part[blockIdx.x] = make_float2(big, total);
}

template <typename T, typename TO, bool VEC>
__global__ void __launch_bounds__(kThreads) softmax_seg_write(const T* __restrict__ x, TO* __restrict__ y, const float2* __restrict__ part,
                                                              float* __restrict__ row_max, float* __restrict__ row_sum, int64_t cols,
                                                              int segs, int64_t seg_len) {
  __shared__ float slots[2][32];
  const Seg g = my_segment(cols, segs, seg_len);
  wait_for_previous_launch();
  float m = -INFINITY, s = 0.0f;
  for (int i = threadIdx.x; i < segs; i += kThreads) {
    const float2 p = __ldcg(&part[g.row * segs + i]);
    const float mn = max_nan(m, p.x);
    s = s * rescale(m, mn) + p.y * rescale(p.x, mn);
    m = mn;
  }
  const float big = block_reduce<MaxOp>(m, slots[0]);
  const float total = block_reduce<SumOp>(s * rescale(m, big), slots[1]);
  const float inv = 1.0f / total;
  const T* xr = x + g.row * cols;
  TO* yr = y + g.row * cols;
  if (VEC) {
#pragma unroll 4
    for (int64_t c = g.c0 + 4 * threadIdx.x; c < g.c1; c += 4 * kThreads) {
      float v[4];
      load4<T>(xr + c, v);
#pragma unroll
      for (int k = 0; k < 4; ++k) v[k] = fast_exp(v[k] - big) * inv;
      store4<TO>(yr + c, v);
    }
  } else {
    for (int64_t c = g.c0 + threadIdx.x; c < g.c1; c += kThreads) yr[c] = from_f32<TO>(fast_exp(to_f32<T>(xr[c]) - big) * inv);
  }
  if (g.c0 == 0 && threadIdx.x == 0) {
    if (row_max) row_max[g.row] = big;
    if (row_sum) row_sum[g.row] = total;
  }
}

// ---- normalisation ---------------------------------------------------------------------------
struct Moments {
  float n, mean, m2;
};
// (n, mean, M2) of the union of two disjoint sets (Chan, Golub, LeVeque)
__device__ __forceinline__ Moments merge(const Moments& a, const Moments& b) {
  if (b.n == 0.0f) return a;
  if (a.n == 0.0f) return b;
  Moments r;
  r.n = a.n + b.n;
  const float d = b.mean - a.mean, f = b.n / r.n;
  r.mean = a.mean + d * f;
  r.m2 = a.m2 + b.m2 + d * d * a.n * f;
  return r;
}
// every thread ends up with the merge of all threads' moments, merged in one fixed tree
__device__ __forceinline__ Moments block_merge(Moments v, float (*slots)[3]) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    Moments other;
    other.n = __shfl_down_sync(0xffffffffu, v.n, o);
    other.mean = __shfl_down_sync(0xffffffffu, v.mean, o);
    other.m2 = __shfl_down_sync(0xffffffffu, v.m2, o);
    v = merge(v, other);
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) { slots[warp][0] = v.n; slots[warp][1] = v.mean; slots[warp][2] = v.m2; }
  __syncthreads();
  Moments r{0.0f, 0.0f, 0.0f};
  for (int w = 0; w < kThreads / 32; ++w) r = merge(r, Moments{slots[w][0], slots[w][1], slots[w][2]});
  return r;
}

// One pass over the segment.  Each thread keeps the sums of (x - pivot) and (x - pivot)^2 with its own first
// element as the pivot — a sample of the data, so the squares stay of the size of the variance and nothing
// cancels — and turns them into (n, mean, M2); the threads' moments are then merged pairwise.
template <typename T, bool VEC>
__global__ void __launch_bounds__(kThreads) norm_seg_stats(const T* __restrict__ x, float2* __restrict__ part, int64_t cols, int segs,
                                                           int64_t seg_len, int centre) {
  __shared__ float slots[kThreads / 32][3];
  const Seg g = my_segment(cols, segs, seg_len);
  let_next_launch_start();
  const T* xr = x + g.row * cols;
  float pivot = 0.0f, ds = 0.0f, dq = 0.0f, n = 0.0f;
  if (VEC) {
    const int64_t first = g.c0 + 4 * threadIdx.x;
    if (centre && first < g.c1) pivot = to_f32<T>(xr[first]);
#pragma unroll 4
    for (int64_t c = first; c < g.c1; c += 4 * kThreads) {
      float v[4];
      load4<T>(xr + c, v);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float d = v[k] - pivot;
        ds += d;
        dq += d * d;
      }
      n += 4.0f;
    }
  } else {
    const int64_t first = g.c0 + threadIdx.x;
    if (centre && first < g.c1) pivot = to_f32<T>(xr[first]);
    for (int64_t c = first; c < g.c1; c += kThreads) {
      const float d = to_f32<T>(xr[c]) - pivot;
      ds += d;
      dq += d * d;
      n += 1.0f;
    }
  }
  Moments mine{n, 0.0f, 0.0f};
  if (n > 0.0f) {
    if (centre) {
      const float dm = ds / n;
      mine.mean = pivot + dm;
      mine.m2 = fmaxf(dq - ds * dm, 0.0f);
    } else {
      mine.m2 = dq;  // rms-norm: deviations from zero, the mean is not subtracted
    }
  }
  Moments all;
  if (centre) {
    all = block_merge(mine, slots);
  } else {  // plain sum of squares
    __shared__ float sq[32];
    all.mean = 0.0f;
    all.m2 = block_reduce<SumOp>(mine.m2, sq);
  }
  if (threadIdx.x == 0) part[blockIdx.x] = make_float2(all.mean, all.m2);
}

template <typename T, typename TW, bool VEC, int AFF>
__global__ void __launch_bounds__(kThreads) norm_seg_write(const T* __restrict__ x, const TW* __restrict__ w, const TW* __restrict__ b,
                                                           T* __restrict__ y, const float2* __restrict__ part, float* __restrict__ mean_out,
                                                           float* __restrict__ rstd_out, int64_t cols, int segs, int64_t seg_len, float eps,
                                                           int64_t inner, int64_t period) {
  __shared__ float slots[kThreads / 32][3];
  const Seg g = my_segment(cols, segs, seg_len);
  wait_for_previous_launch();
  Moments mine{0.0f, 0.0f, 0.0f};
  for (int i = threadIdx.x; i < segs; i += kThreads) {  // segments i, i + 512, ... in order
    const float2 p = __ldcg(&part[g.row * segs + i]);
    const int64_t a = (int64_t)i * seg_len, e = a + seg_len < cols ? a + seg_len : cols;
    mine = merge(mine, Moments{(float)(e - a), p.x, p.y});
  }
  const Moments all = block_merge(mine, slots);
  const float mean = all.mean, rstd = 1.0f / sqrtf(all.m2 / (float)cols + eps);
  const T* xr = x + g.row * cols;
  T* yr = y + g.row * cols;
  auto affine_index = [&](int64_t c) -> int64_t { return AFF == AFF_COL ? c : ((g.row * cols + c) / inner) % period; };
  if (VEC) {
#pragma unroll 2
    for (int64_t c = g.c0 + 4 * threadIdx.x; c < g.c1; c += 4 * kThreads) {
      float v[4], wv[4] = {1.f, 1.f, 1.f, 1.f}, bv[4] = {0.f, 0.f, 0.f, 0.f};
      load4<T>(xr + c, v);
      if (AFF == AFF_COL) {
        if (w) load4<TW>(w + c, wv);
        if (b) load4<TW>(b + c, bv);
      } else if (AFF == AFF_GENERIC) {
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const int64_t idx = affine_index(c + k);
          if (w) wv[k] = to_f32<TW>(w[idx]);
          if (b) bv[k] = to_f32<TW>(b[idx]);
        }
      }
#pragma unroll
      for (int k = 0; k < 4; ++k) v[k] = (v[k] - mean) * rstd * wv[k] + bv[k];
      store4<T>(yr + c, v);
    }
  } else {
    for (int64_t c = g.c0 + threadIdx.x; c < g.c1; c += kThreads) {
      float wv = 1.0f, bv = 0.0f;
      if (AFF != AFF_NONE) {
        const int64_t idx = affine_index(c);
        if (w) wv = to_f32<TW>(w[idx]);
        if (b) bv = to_f32<TW>(b[idx]);
      }
      yr[c] = from_f32<T>((to_f32<T>(xr[c]) - mean) * rstd * wv + bv);
    }
  }
  if (g.c0 == 0 && threadIdx.x == 0) {
    if (mean_out) mean_out[g.row] = mean;
    if (rstd_out) rstd_out[g.row] = rstd;
  }
}

// ---- the whole tensor resident in shared memory: one launch -----------------------------------------------------
// When rows x cols fits into the shared memory of the GPU (29 MB: [4, 1 Mi] f32 does), the two passes become one
// kernel: a CTA copies its segment into shared memory while it reduces it, publishes its pair of statistics, waits
// until the pairs of its row are all there, and writes its segment from shared memory.  x is read from HBM once and
// nothing is launched twice.  The CTAs of a row wait for one another, so the kernel is launched cooperatively (the
// runtime refuses the launch unless all CTAs are resident at once), the counter they meet at is zeroed in front of
// the launch, and the wait is bounded: when it runs out the CTA records status 7 and finishes with what it has.
template <typename T> struct Raw4 { using type = uint2; };
template <> struct Raw4<float> { using type = float4; };

constexpr uint32_t kMeetLimit = 1u << 21;  // polls of ~0.1 us and more each: a fraction of a second

__device__ __forceinline__ uint32_t load_acquire(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// thread 0 publishes this CTA's arrival and waits for the row's other CTAs; everybody leaves together
__device__ __forceinline__ void meet_row(uint32_t* counter, uint32_t parties, int32_t* status) {
  if (threadIdx.x == 0) {
    __threadfence();
    atomicAdd(counter, 1u);
    uint32_t polls = 0;
    while (load_acquire(counter) < parties) {
      if (++polls > kMeetLimit) {
        if (status) atomicCAS(status, 0, 7);
        break;
      }
      __nanosleep(64);
    }
  }
  __syncthreads();
}

template <typename T, typename TO>
__global__ void __launch_bounds__(kThreads, 1) softmax_resident(const T* __restrict__ x, TO* __restrict__ y, float2* __restrict__ part,
                                                               uint32_t* __restrict__ counters, float* __restrict__ row_max,
                                                               float* __restrict__ row_sum, int64_t cols, int segs, int64_t seg_len,
                                                               int32_t* status) {
  extern __shared__ __align__(16) unsigned char seg_mem[];
  __shared__ float slots[2][32];
  using Raw = typename Raw4<T>::type;
  T* mine = reinterpret_cast<T*>(seg_mem);
  const Seg g = my_segment(cols, segs, seg_len);
  const int n = (int)(g.c1 - g.c0);
  const T* xr = x + g.row * cols + g.c0;
  float m = -INFINITY, s = 0.0f;
#pragma unroll 4
  for (int c = 4 * threadIdx.x; c < n; c += 4 * kThreads) {
    const Raw raw = *reinterpret_cast<const Raw*>(xr + c);
    *reinterpret_cast<Raw*>(mine + c) = raw;
    float v[4];
    load4<T>(reinterpret_cast<const T*>(&raw), v);
    const float mn = max_nan(m, max_nan(max_nan(v[0], v[1]), max_nan(v[2], v[3])));
    float add = 0.0f;
    if (mn != -INFINITY) add = fast_exp(v[0] - mn) + fast_exp(v[1] - mn) + fast_exp(v[2] - mn) + fast_exp(v[3] - mn);
    s = s * rescale(m, mn) + add;
    m = mn;
  }
  float big = block_reduce<MaxOp>(m, slots[0]);
  float total = block_reduce<SumOp>(s * rescale(m, big), slots[1]);
  if (threadIdx.x == 0) part[blockIdx.x] = make_float2(big, total);
  meet_row(counters + g.row, (uint32_t)segs, status);
  m = -INFINITY, s = 0.0f;
  for (int i = threadIdx.x; i < segs; i += kThreads) {
    const float2 p = __ldcg(&part[g.row * segs + i]);
    const float mn = max_nan(m, p.x);
    s = s * rescale(m, mn) + p.y * rescale(p.x, mn);
    m = mn;
  }
  big = block_reduce<MaxOp>(m, slots[0]);
  total = block_reduce<SumOp>(s * rescale(m, big), slots[1]);
  const float inv = 1.0f / total;
  TO* yr = y + g.row * cols + g.c0;
#pragma unroll 4
  for (int c = 4 * threadIdx.x; c < n; c += 4 * kThreads) {
    float v[4];
    load4<T>(mine + c, v);
#pragma unroll
    for (int k = 0; k < 4; ++k) v[k] = fast_exp(v[k] - big) * inv;
    store4<TO>(yr + c, v);
  }
  if (g.c0 == 0 && threadIdx.x == 0) {
    if (row_max) row_max[g.row] = big;
    if (row_sum) row_sum[g.row] = total;
  }
}

template <typename T, typename TW, int AFF>
__global__ void __launch_bounds__(kThreads, 1) norm_resident(const T* __restrict__ x, const TW* __restrict__ w, const TW* __restrict__ b,
                                                            T* __restrict__ y, float2* __restrict__ part, uint32_t* __restrict__ counters,
                                                            float* __restrict__ mean_out, float* __restrict__ rstd_out, int64_t cols, int segs,
                                                            int64_t seg_len, float eps, int64_t inner, int64_t period, int centre,
                                                            int32_t* status) {
  extern __shared__ __align__(16) unsigned char seg_mem[];
  __shared__ float slots[kThreads / 32][3];
  __shared__ float sq[32];
  using Raw = typename Raw4<T>::type;
  T* mine = reinterpret_cast<T*>(seg_mem);
  const Seg g = my_segment(cols, segs, seg_len);
  const int n = (int)(g.c1 - g.c0);
  const T* xr = x + g.row * cols + g.c0;
  float pivot = 0.0f, ds = 0.0f, dq = 0.0f, cnt = 0.0f;
  if (centre && 4 * (int)threadIdx.x < n) pivot = to_f32<T>(xr[4 * threadIdx.x]);
#pragma unroll 4
  for (int c = 4 * threadIdx.x; c < n; c += 4 * kThreads) {
    const Raw raw = *reinterpret_cast<const Raw*>(xr + c);
    *reinterpret_cast<Raw*>(mine + c) = raw;
    float v[4];
    load4<T>(reinterpret_cast<const T*>(&raw), v);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float d = v[k] - pivot;
      ds += d;
      dq += d * d;
    }
    cnt += 4.0f;
  }
  Moments own{cnt, 0.0f, 0.0f};
  if (cnt > 0.0f) {
    if (centre) {
      const float dm = ds / cnt;
      own.mean = pivot + dm;
      own.m2 = fmaxf(dq - ds * dm, 0.0f);
    } else {
      own.m2 = dq;
    }
  }
  Moments all;
  if (centre) {
    all = block_merge(own, slots);
  } else {
    all.mean = 0.0f;
    all.m2 = block_reduce<SumOp>(own.m2, sq);
  }
  if (threadIdx.x == 0) part[blockIdx.x] = make_float2(all.mean, all.m2);
  meet_row(counters + g.row, (uint32_t)segs, status);
  Moments fold{0.0f, 0.0f, 0.0f};
  for (int i = threadIdx.x; i < segs; i += kThreads) {
    const float2 p = __ldcg(&part[g.row * segs + i]);
    const int64_t a = (int64_t)i * seg_len, e = a + seg_len < cols ? a + seg_len : cols;
    fold = merge(fold, Moments{(float)(e - a), p.x, p.y});
  }
  all = block_merge(fold, slots);
  const float mean = all.mean, rstd = 1.0f / sqrtf(all.m2 / (float)cols + eps);
  T* yr = y + g.row * cols + g.c0;
#pragma unroll 2
  for (int c = 4 * threadIdx.x; c < n; c += 4 * kThreads) {
    float v[4], wv[4] = {1.f, 1.f, 1.f, 1.f}, bv[4] = {0.f, 0.f, 0.f, 0.f};
    load4<T>(mine + c, v);
    if (AFF == AFF_COL) {
      if (w) load4<TW>(w + g.c0 + c, wv);
      if (b) load4<TW>(b + g.c0 + c, bv);
    } else if (AFF == AFF_GENERIC) {
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const int64_t idx = ((g.row * cols + g.c0 + c + k) / inner) % period;
        if (w) wv[k] = to_f32<TW>(w[idx]);
        if (b) bv[k] = to_f32<TW>(b[idx]);
      }
    }
#pragma unroll
    for (int k = 0; k < 4; ++k) v[k] = (v[k] - mean) * rstd * wv[k] + bv[k];
    store4<T>(yr + c, v);
  }
  if (g.c0 == 0 && threadIdx.x == 0) {
    if (mean_out) mean_out[g.row] = mean;
    if (rstd_out) rstd_out[g.row] = rstd;
  }
}

struct SegPlan {
  int segs;
  int64_t seg_len;
};

// launch `kernel` so that it may begin while the launch in front of it on the stream is finishing
template <typename... KArgs, typename... Args>
cudaError_t launch_dependent(void (*kernel)(KArgs...), unsigned grid, cudaStream_t s, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(kThreads);
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// Segments per row: enough CTAs for four per SM, segments of 8 Ki .. 64 Ki elements (whole multiples of 2048, so
// that every segment starts on a vector boundary of its row).
bool plan_segments(int64_t rows, int64_t cols, int elem_bytes, int64_t resident_limit, SegPlan* out) {
  if (rows <= 0 || cols <= resident_limit) return false;  // the register- / cluster-resident kernels cover the row
  // one streaming CTA per row is fine while there are rows enough to fill the GPU and the rows it works on fit L2
  const int64_t active = rows < 2 * kSmCount ? rows : 2 * kSmCount;
  const bool rows_fill_gpu = rows >= 2 * kSmCount, rows_fit_l2 = active * cols * elem_bytes <= ((int64_t)64 << 20);
  if (rows_fill_gpu && rows_fit_l2) return false;
  int64_t segs = (4 * (int64_t)kSmCount + rows - 1) / rows;
  if (segs < (cols + kMaxSeg - 1) / kMaxSeg) segs = (cols + kMaxSeg - 1) / kMaxSeg;
  int64_t len = (cols + segs - 1) / segs;
  if (len < kMinSeg) len = kMinSeg;
  len = (len + 2047) / 2048 * 2048;
  segs = (cols + len - 1) / len;
  if (segs < 2 || segs > kMaxSegs || rows * segs >= ((int64_t)1 << 31)) return false;
  out->segs = (int)segs;
  out->seg_len = len;
  return true;
}

// The one-launch form: as many segments per row as there are SMs for it, each at most what one CTA can keep in
// shared memory beside its static arrays.
constexpr size_t kResidentBytes = 200 * 1024;
bool plan_resident(int64_t rows, int64_t cols, int elem_bytes, SegPlan* out) {
  if (rows <= 0 || rows > kSmCount / 2 || cols % 8 != 0) return false;
  int64_t segs = kSmCount / rows;
  int64_t len = (cols + segs - 1) / segs;
  if (len < 2048) len = 2048;
  len = (len + 7) / 8 * 8;  // every segment starts on a 16-byte boundary for 2- and 4-byte elements
  segs = (cols + len - 1) / len;
  if (segs < 2 || (size_t)len * elem_bytes > kResidentBytes) return false;
  out->segs = (int)segs;
  out->seg_len = len;
  return true;
}
size_t resident_scratch_bytes(int64_t rows, const SegPlan& rp) { return ((size_t)rows * rp.segs * sizeof(float2) + 15) / 16 * 16 + (size_t)rows * 4; }
// what the segmented forms of one shape need: the pairs of the two-launch form, or the pairs and the meeting
// counters of the one-launch form, whichever is more
size_t long_row_scratch(int64_t rows, int64_t cols, int elem_bytes, const SegPlan& sp) {
  size_t bytes = (size_t)rows * sp.segs * sizeof(float2);
  SegPlan rp;
  if (plan_resident(rows, cols, elem_bytes, &rp) && resident_scratch_bytes(rows, rp) > bytes) bytes = resident_scratch_bytes(rows, rp);
  return bytes;
}

// launches `kernel` cooperatively with `smem` bytes of dynamic shared memory; false (nothing launched, no error left
// behind) when the grid cannot be resident at once or the launch is refused
template <typename... KArgs, typename... Args>
bool launch_resident(void (*kernel)(KArgs...), unsigned grid, size_t smem, cudaStream_t s, Args... args) {
  static std::mutex mu;
  static std::map<std::tuple<const void*, size_t, int>, int> fits;  // (kernel, smem, device) -> CTAs per SM
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) { cudaGetLastError(); return false; }
  int per_sm = 0;
  {
    std::lock_guard<std::mutex> lock(mu);
    const auto key = std::make_tuple(reinterpret_cast<const void*>(kernel), smem, dev);
    auto it = fits.find(key);
    if (it == fits.end()) {
      int n = 0;
      if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kResidentBytes) != cudaSuccess ||
          cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kernel, kThreads, smem) != cudaSuccess) {
        cudaGetLastError();
        n = 0;
      }
      it = fits.emplace(key, n).first;
    }
    per_sm = it->second;
  }
  if (per_sm < 1 || grid > (unsigned)(per_sm * kSmCount)) return false;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeCooperative;
  attr[0].val.cooperative = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...) != cudaSuccess) {
    cudaGetLastError();
    return false;
  }
  return true;
}

}  // namespace

size_t softmax_scratch_bytes(int64_t rows, int64_t cols, int elem_bytes) {
  SegPlan sp;
  return plan_segments(rows, cols, elem_bytes, 16384, &sp) ? long_row_scratch(rows, cols, elem_bytes, sp) : 0;
}
// normalisation has cluster kernels for rows of up to 128 Ki elements: those rows are segmented only when there are
// too few of them for the clusters to matter (8 CTAs per row)
static bool plan_norm_segments(int64_t rows, int64_t cols, int elem_bytes, SegPlan* sp) {
  if (plan_segments(rows, cols, elem_bytes, 131072, sp)) return true;
  return cols > 16384 && rows * 8 < kSmCount && plan_segments(rows, cols, elem_bytes, 16384, sp);
}
size_t norm_scratch_bytes(int64_t rows, int64_t cols, int elem_bytes) {
  SegPlan sp;
  return plan_norm_segments(rows, cols, elem_bytes, &sp) ? long_row_scratch(rows, cols, elem_bytes, sp) : 0;
}

template <typename T, typename TO>
static int softmax_segmented(const void* xv, void* yv, float* mx, float* sm, int64_t rows, int64_t cols, const SegPlan& sp, void* scratch,
                             size_t scratch_bytes, cudaStream_t s, int32_t* status) {
  const T* x = static_cast<const T*>(xv);
  TO* y = static_cast<TO*>(yv);
  float2* part = static_cast<float2*>(scratch);
  const bool vec = aligned16(x) && aligned16(y) && cols % 4 == 0;
  SegPlan rp;
  if (vec && plan_resident(rows, cols, (int)sizeof(T), &rp) && resident_scratch_bytes(rows, rp) <= scratch_bytes) {
    uint32_t* counters = reinterpret_cast<uint32_t*>(static_cast<char*>(scratch) + ((size_t)rows * rp.segs * sizeof(float2) + 15) / 16 * 16);
    if (cudaMemsetAsync(counters, 0, (size_t)rows * 4, s) != cudaSuccess) return cuda_fail(cudaGetLastError(), "segmented softmax: counters");
    if (launch_resident(softmax_resident<T, TO>, (unsigned)(rows * rp.segs), (size_t)rp.seg_len * sizeof(T), s, x, y, part, counters, mx, sm, cols,
                        rp.segs, rp.seg_len, status))
      return IB200_OK;
  }
  const unsigned grid = (unsigned)(rows * sp.segs);
  if (vec) {
    softmax_seg_stats<T, true><<<grid, kThreads, 0, s>>>(x, part, cols, sp.segs, sp.seg_len);
    launch_dependent(softmax_seg_write<T, TO, true>, grid, s, x, y, part, mx, sm, cols, sp.segs, sp.seg_len);
  } else {
    softmax_seg_stats<T, false><<<grid, kThreads, 0, s>>>(x, part, cols, sp.segs, sp.seg_len);
    launch_dependent(softmax_seg_write<T, TO, false>, grid, s, x, y, part, mx, sm, cols, sp.segs, sp.seg_len);
  }
  return cudaPeekAtLastError() == cudaSuccess ? IB200_OK : cuda_fail(cudaGetLastError(), "segmented softmax launch");
}

// Returns IB200_OK after launching, or 1 when the shape is not a long-row case / the scratch is too small
// (the caller then uses the ordinary kernels).
int try_softmax_segmented(const void* x, void* y, float* row_max, float* row_sum, int dtype, int out_dtype, int64_t rows, int64_t cols,
                          void* scratch, size_t scratch_bytes, cudaStream_t s, int32_t* status) {
  SegPlan sp;
  const int esz = dtype == IB200_F32 ? 4 : 2;
  if (!scratch || !plan_segments(rows, cols, esz, 16384, &sp) || scratch_bytes < (size_t)rows * sp.segs * sizeof(float2)) return 1;
  if (!status) status = norm_default_status();
#define IB200_S(T, TO) return softmax_segmented<T, TO>(x, y, row_max, row_sum, rows, cols, sp, scratch, scratch_bytes, s, status)
  if (dtype == IB200_F32 && out_dtype == IB200_F32) IB200_S(float, float);
  if (dtype == IB200_BF16 && out_dtype == IB200_BF16) IB200_S(__nv_bfloat16, __nv_bfloat16);
  if (dtype == IB200_F16 && out_dtype == IB200_F16) IB200_S(__half, __half);
  if (dtype == IB200_BF16 && out_dtype == IB200_F32) IB200_S(__nv_bfloat16, float);
  if (dtype == IB200_F16 && out_dtype == IB200_F32) IB200_S(__half, float);
#undef IB200_S
  return 1;
}

template <typename T, typename TW>
static int norm_segmented(const void* xv, const void* wv, const void* bv, void* yv, float* mean, float* rstd, int64_t rows, int64_t cols,
                          int64_t inner, int64_t period, float eps, int centre, const SegPlan& sp, void* scratch, size_t scratch_bytes,
                          cudaStream_t s, int32_t* status) {
  const T* x = static_cast<const T*>(xv);
  T* y = static_cast<T*>(yv);
  const TW* w = static_cast<const TW*>(wv);
  const TW* b = static_cast<const TW*>(bv);
  float2* part = static_cast<float2*>(scratch);
  bool vec = aligned16(x) && aligned16(y) && cols % 4 == 0;
  const int aff = (!w && !b) ? AFF_NONE : (inner == 1 && period == cols) ? AFF_COL : AFF_GENERIC;
  if (aff == AFF_COL && vec) vec = (!w || aligned16(w)) && (!b || aligned16(b));
  SegPlan rp;
  if (vec && plan_resident(rows, cols, (int)sizeof(T), &rp) && resident_scratch_bytes(rows, rp) <= scratch_bytes) {
    uint32_t* counters = reinterpret_cast<uint32_t*>(static_cast<char*>(scratch) + ((size_t)rows * rp.segs * sizeof(float2) + 15) / 16 * 16);
    if (cudaMemsetAsync(counters, 0, (size_t)rows * 4, s) != cudaSuccess) return cuda_fail(cudaGetLastError(), "segmented norm: counters");
    const unsigned rgrid = (unsigned)(rows * rp.segs);
    const size_t smem = (size_t)rp.seg_len * sizeof(T);
#define IB200_R(A) launch_resident(norm_resident<T, TW, A>, rgrid, smem, s, x, w, b, y, part, counters, mean, rstd, cols, rp.segs, rp.seg_len, eps, inner, period, centre, status)
    const bool launched = aff == AFF_NONE ? IB200_R(AFF_NONE) : aff == AFF_COL ? IB200_R(AFF_COL) : IB200_R(AFF_GENERIC);
#undef IB200_R
    if (launched) return IB200_OK;
  }
  const unsigned grid = (unsigned)(rows * sp.segs);
  if (vec) norm_seg_stats<T, true><<<grid, kThreads, 0, s>>>(x, part, cols, sp.segs, sp.seg_len, centre);
  else norm_seg_stats<T, false><<<grid, kThreads, 0, s>>>(x, part, cols, sp.segs, sp.seg_len, centre);
#define IB200_W(V, A) launch_dependent(norm_seg_write<T, TW, V, A>, grid, s, x, w, b, y, part, mean, rstd, cols, sp.segs, sp.seg_len, eps, inner, period)
  if (vec) {
    if (aff == AFF_NONE) IB200_W(true, AFF_NONE); else if (aff == AFF_COL) IB200_W(true, AFF_COL); else IB200_W(true, AFF_GENERIC);
  } else {
    if (aff == AFF_NONE) IB200_W(false, AFF_NONE); else if (aff == AFF_COL) IB200_W(false, AFF_COL); else IB200_W(false, AFF_GENERIC);
  }
#undef IB200_W
  return cudaPeekAtLastError() == cudaSuccess ? IB200_OK : cuda_fail(cudaGetLastError(), "segmented norm launch");
}

int try_norm_segmented(const void* x, const void* w, const void* b, void* y, float* mean, float* rstd, int dtype, int affine_dtype,
                       int64_t rows, int64_t cols, int64_t inner, int64_t period, float eps, int centre, void* scratch, size_t scratch_bytes,
                       cudaStream_t s, int32_t* status) {
  SegPlan sp;
  const int esz = dtype == IB200_F32 ? 4 : 2;
  if (!scratch || !plan_norm_segments(rows, cols, esz, &sp)) return 1;
  if (scratch_bytes < (size_t)rows * sp.segs * sizeof(float2)) return 1;
  if ((w || b) && (inner < 1 || period < 1)) return 1;
  const int adt = (w || b) ? affine_dtype : dtype;
  if (!status) status = norm_default_status();
#define IB200_N(T, TW) return norm_segmented<T, TW>(x, w, b, y, mean, rstd, rows, cols, inner, period, eps, centre, sp, scratch, scratch_bytes, s, status)
  if (dtype == IB200_F32 && adt == IB200_F32) IB200_N(float, float);
  if (dtype == IB200_BF16 && adt == IB200_BF16) IB200_N(__nv_bfloat16, __nv_bfloat16);
  if (dtype == IB200_BF16 && adt == IB200_F32) IB200_N(__nv_bfloat16, float);
  if (dtype == IB200_F16 && adt == IB200_F16) IB200_N(__half, __half);
  if (dtype == IB200_F16 && adt == IB200_F32) IB200_N(__half, float);
#undef IB200_N
  return 1;
}

}  // namespace ib200
