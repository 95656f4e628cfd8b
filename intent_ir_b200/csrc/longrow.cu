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

enum { AFF_NONE = 0, AFF_COL = 1, AFF_GENERIC = 2 };

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

}  // namespace

size_t softmax_scratch_bytes(int64_t rows, int64_t cols, int elem_bytes) {
  SegPlan sp;
  return plan_segments(rows, cols, elem_bytes, 16384, &sp) ? (size_t)rows * sp.segs * sizeof(float2) : 0;
}
// normalisation has cluster kernels for rows of up to 128 Ki elements: those rows are segmented only when there are
// too few of them for the clusters to matter (8 CTAs per row)
static bool plan_norm_segments(int64_t rows, int64_t cols, int elem_bytes, SegPlan* sp) {
  if (plan_segments(rows, cols, elem_bytes, 131072, sp)) return true;
  return cols > 16384 && rows * 8 < kSmCount && plan_segments(rows, cols, elem_bytes, 16384, sp);
}
size_t norm_scratch_bytes(int64_t rows, int64_t cols, int elem_bytes) {
  SegPlan sp;
  return plan_norm_segments(rows, cols, elem_bytes, &sp) ? (size_t)rows * sp.segs * sizeof(float2) : 0;
}

template <typename T, typename TO>
static int softmax_segmented(const void* xv, void* yv, float* mx, float* sm, int64_t rows, int64_t cols, const SegPlan& sp, void* scratch,
                             cudaStream_t s) {
  const T* x = static_cast<const T*>(xv);
  TO* y = static_cast<TO*>(yv);
  float2* part = static_cast<float2*>(scratch);
  const bool vec = aligned16(x) && aligned16(y) && cols % 4 == 0;
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
                          void* scratch, size_t scratch_bytes, cudaStream_t s) {
  SegPlan sp;
  const int esz = dtype == IB200_F32 ? 4 : 2;
  if (!scratch || !plan_segments(rows, cols, esz, 16384, &sp) || scratch_bytes < (size_t)rows * sp.segs * sizeof(float2)) return 1;
  if (dtype == IB200_F32 && out_dtype == IB200_F32) return softmax_segmented<float, float>(x, y, row_max, row_sum, rows, cols, sp, scratch, s);
  if (dtype == IB200_BF16 && out_dtype == IB200_BF16) return softmax_segmented<__nv_bfloat16, __nv_bfloat16>(x, y, row_max, row_sum, rows, cols, sp, scratch, s);
  if (dtype == IB200_F16 && out_dtype == IB200_F16) return softmax_segmented<__half, __half>(x, y, row_max, row_sum, rows, cols, sp, scratch, s);
  if (dtype == IB200_BF16 && out_dtype == IB200_F32) return softmax_segmented<__nv_bfloat16, float>(x, y, row_max, row_sum, rows, cols, sp, scratch, s);
  if (dtype == IB200_F16 && out_dtype == IB200_F32) return softmax_segmented<__half, float>(x, y, row_max, row_sum, rows, cols, sp, scratch, s);
  return 1;
}

template <typename T, typename TW>
static int norm_segmented(const void* xv, const void* wv, const void* bv, void* yv, float* mean, float* rstd, int64_t rows, int64_t cols,
                          int64_t inner, int64_t period, float eps, int centre, const SegPlan& sp, void* scratch, cudaStream_t s) {
  const T* x = static_cast<const T*>(xv);
  T* y = static_cast<T*>(yv);
  const TW* w = static_cast<const TW*>(wv);
  const TW* b = static_cast<const TW*>(bv);
  float2* part = static_cast<float2*>(scratch);
  bool vec = aligned16(x) && aligned16(y) && cols % 4 == 0;
  const int aff = (!w && !b) ? AFF_NONE : (inner == 1 && period == cols) ? AFF_COL : AFF_GENERIC;
  if (aff == AFF_COL && vec) vec = (!w || aligned16(w)) && (!b || aligned16(b));
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
                       cudaStream_t s) {
  SegPlan sp;
  const int esz = dtype == IB200_F32 ? 4 : 2;
  if (!scratch || !plan_norm_segments(rows, cols, esz, &sp)) return 1;
  if (scratch_bytes < (size_t)rows * sp.segs * sizeof(float2)) return 1;
  if ((w || b) && (inner < 1 || period < 1)) return 1;
  const int adt = (w || b) ? affine_dtype : dtype;
#define IB200_N(T, TW) return norm_segmented<T, TW>(x, w, b, y, mean, rstd, rows, cols, inner, period, eps, centre, sp, scratch, s)
  if (dtype == IB200_F32 && adt == IB200_F32) IB200_N(float, float);
  if (dtype == IB200_BF16 && adt == IB200_BF16) IB200_N(__nv_bfloat16, __nv_bfloat16);
  if (dtype == IB200_BF16 && adt == IB200_F32) IB200_N(__nv_bfloat16, float);
  if (dtype == IB200_F16 && adt == IB200_F16) IB200_N(__half, __half);
  if (dtype == IB200_F16 && adt == IB200_F32) IB200_N(__half, float);
#undef IB200_N
  return 1;
}

}  // namespace ib200
