// Axis reductions: out[o, i] = reduce_r x[o, r, i] for sum (with optional scale), max
// (NaN-propagating, like np.max) and any (element != 0).  HBM-bound: every input byte is
// read exactly once with 128-bit loads where the layout allows, partial results live in
// registers and are combined with warp shuffles.
//
//   inner == 1 (reduction over the trailing axes):
//     rows_warp  : one warp per row, for rows of up to 2048 elements;
//     rows_block : one 256-thread CTA per row for longer rows.
//     rows_split : fewer rows than two per SM and rows of 64 Ki elements or more: every row is cut
//                  into segments, one CTA each; a CTA leaves its partial in a scratch area and takes a
//                  ticket from the row's counter, and the CTA that draws the last ticket folds the
//                  partials in segment order (same result on every run).  Nobody waits for anybody.
//                  Needs a scratch area from the caller (plans provide it); the launcher zeroes the
//                  counters with a memset node in front of the kernel, so the area may be shared.
//   inner  > 1 (reduction over a leading / middle axis):
//     cols_vec   : inner % 4 == 0: a CTA covers 4*L adjacent inner positions (L = 8, 16 or 32 lanes, each
//                  with one 128-bit load per row) and 256/L rows at a time, four rows in flight per
//                  thread; the thread rows are combined through shared memory.  When the results alone
//                  give too few CTAs the reduced axis is cut into segments, folded as in rows_split.
//     cols       : any inner: a 32x8 CTA covers 32 adjacent inner positions; the 8 thread rows stride
//                  over the reduced axis and are combined through shared memory.
//
// Semantics follow verify/interpreter.py:478-500 of the reference (np.sum / np.max / np.any).
#include "common.cuh"

namespace ib200 {
namespace {

template <int KIND> struct KindOp;
template <> struct KindOp<IB200_REDUCE_SUM> { using Op = SumOp; };
template <> struct KindOp<IB200_REDUCE_MAX> { using Op = MaxOp; };
template <> struct KindOp<IB200_REDUCE_ANY> { using Op = AnyOp; };

template <int KIND> __device__ __forceinline__ float prep(float v) {
  return KIND == IB200_REDUCE_ANY ? (v != 0.0f ? 1.0f : 0.0f) : v;
}

template <typename TO> __device__ __forceinline__ void write_result(TO* out, int64_t i, float v, float scale, int kind) {
  if (kind == IB200_REDUCE_SUM) v *= scale;
  out[i] = from_f32<TO>(v);
}

// accumulate one row segment [0, n) starting at p into 4 independent partials
template <typename T, int KIND, bool VEC>
__device__ __forceinline__ float row_partial(const T* __restrict__ p, int64_t n, int tid, int nthreads) {
  using Op = typename KindOp<KIND>::Op;
  float acc[4] = {Op::identity(), Op::identity(), Op::identity(), Op::identity()};
  if (VEC) {
    const int64_t nvec = n >> 2;
    int64_t i = tid;
    // four 128-bit loads in flight per thread per iteration while the row lasts, then two, then one
    for (; i + 3 * (int64_t)nthreads < nvec; i += 4 * (int64_t)nthreads) {
      float a[4][4];
#pragma unroll
      for (int u = 0; u < 4; ++u) load4<T>(p + 4 * (i + u * (int64_t)nthreads), a[u]);
#pragma unroll
      for (int k = 0; k < 4; ++k)
        acc[k] = Op::apply(Op::apply(Op::apply(acc[k], prep<KIND>(a[0][k])), prep<KIND>(a[1][k])), Op::apply(prep<KIND>(a[2][k]), prep<KIND>(a[3][k])));
    }
    for (; i + nthreads < nvec; i += 2 * (int64_t)nthreads) {
      float a[4], b[4];
      load4<T>(p + 4 * i, a);
      load4<T>(p + 4 * (i + nthreads), b);
#pragma unroll
      for (int k = 0; k < 4; ++k) acc[k] = Op::apply(Op::apply(acc[k], prep<KIND>(a[k])), prep<KIND>(b[k]));
    }
    for (; i < nvec; i += nthreads) {
      float a[4];
      load4<T>(p + 4 * i, a);
#pragma unroll
      for (int k = 0; k < 4; ++k) acc[k] = Op::apply(acc[k], prep<KIND>(a[k]));
    }
  } else {
    int64_t i = tid;
    for (; i + 3 * (int64_t)nthreads < n; i += 4 * (int64_t)nthreads) {
#pragma unroll
      for (int k = 0; k < 4; ++k) acc[k] = Op::apply(acc[k], prep<KIND>(to_f32<T>(p[i + k * (int64_t)nthreads])));
    }
    for (; i < n; i += nthreads) acc[0] = Op::apply(acc[0], prep<KIND>(to_f32<T>(p[i])));
  }
  return Op::apply(Op::apply(acc[0], acc[1]), Op::apply(acc[2], acc[3]));
}

template <typename T, typename TO, int KIND, bool VEC>
__global__ void __launch_bounds__(256) reduce_rows_warp(const T* __restrict__ x, TO* __restrict__ out, int64_t rows,
                                                        int64_t n, float scale) {
  using Op = typename KindOp<KIND>::Op;
  const int lane = threadIdx.x & 31;
  const int64_t warps = (int64_t)gridDim.x * (blockDim.x >> 5);
  for (int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); row < rows; row += warps) {
    float v = warp_reduce<Op>(row_partial<T, KIND, VEC>(x + row * n, n, lane, 32));
    if (lane == 0) write_result<TO>(out, row, v, scale, KIND);
  }
}

// Rows of at most 128 elements: LANES (8 or 16) lanes per row, so a warp works on 4 or 2 rows at a
// time and no lane idles (a whole warp on a 64-element row keeps 16 of its 32 lanes empty and too
// few bytes in flight: measured 0.30 of HBM peak on [1048576, 64]).
template <typename T, typename TO, int KIND, int LANES>
__global__ void __launch_bounds__(256) reduce_rows_sub(const T* __restrict__ x, TO* __restrict__ out, int64_t rows, int n, float scale) {
  using Op = typename KindOp<KIND>::Op;
  const int sub = threadIdx.x % LANES;
  const int64_t groups = (int64_t)gridDim.x * (256 / LANES);
  const int64_t first = (int64_t)blockIdx.x * (256 / LANES) + threadIdx.x / LANES;
  const int nvec = n >> 2;
  const int64_t trips = (rows + groups - 1) / groups;  // the same for every lane: the shuffles below need the whole warp
  for (int64_t it = 0; it < trips; ++it) {
    const int64_t row = first + it * groups;
    float acc[4] = {Op::identity(), Op::identity(), Op::identity(), Op::identity()};
    if (row < rows) {
      const T* p = x + row * n;
      for (int v = sub; v < nvec; v += LANES) {
        float a[4];
        load4<T>(p + 4 * v, a);
#pragma unroll
        for (int k = 0; k < 4; ++k) acc[k] = Op::apply(acc[k], prep<KIND>(a[k]));
      }
    }
    float r = Op::apply(Op::apply(acc[0], acc[1]), Op::apply(acc[2], acc[3]));
#pragma unroll
    for (int o = LANES / 2; o > 0; o >>= 1) r = Op::apply(r, __shfl_xor_sync(0xffffffffu, r, o));
    if (sub == 0 && row < rows) write_result<TO>(out, row, r, scale, KIND);
  }
}

template <typename T, typename TO, int KIND, bool VEC>
__global__ void __launch_bounds__(256) reduce_rows_block(const T* __restrict__ x, TO* __restrict__ out, int64_t rows,
                                                         int64_t n, float scale) {
  using Op = typename KindOp<KIND>::Op;
  __shared__ float slots[2][8];
  int flip = 0;
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x, flip ^= 1) {
    float v = block_reduce<Op>(row_partial<T, KIND, VEC>(x + row * n, n, threadIdx.x, blockDim.x), slots[flip]);
    if (threadIdx.x == 0) write_result<TO>(out, row, v, scale, KIND);
  }
}

constexpr size_t kRowScratchBytes = 8192;
constexpr int kSplitCounters = 512;  // counters (one per row) in front of the partials in the scratch area
constexpr int kSplitPartials = (int)((kRowScratchBytes - kSplitCounters * sizeof(unsigned)) / sizeof(float));
int row_split_factor(int64_t outer, int64_t reduce, int64_t inner);
constexpr int64_t kSplitAlign = 1024;  // segment length granularity in elements: keeps every segment start 16-byte aligned for all types

template <typename T, typename TO, int KIND, bool VEC>
__global__ void __launch_bounds__(256) reduce_rows_split(const T* __restrict__ x, TO* __restrict__ out, int64_t n, int split, int64_t seg,
                                                         float scale, unsigned* __restrict__ counters, float* __restrict__ partials) {
  using Op = typename KindOp<KIND>::Op;
  __shared__ float slots[2][8];
  __shared__ unsigned ticket;
  const int64_t row = blockIdx.x / split;
  const int part = blockIdx.x % split;
  const int64_t lo = (int64_t)part * seg;
  const int64_t len = n - lo < seg ? n - lo : seg;
  const float mine = block_reduce<Op>(row_partial<T, KIND, VEC>(x + row * n + lo, len, threadIdx.x, 256), slots[0]);
  if (threadIdx.x == 0) {
    __stcg(&partials[blockIdx.x], mine);
    __threadfence();  // the partial is visible before the ticket is
    ticket = atomicAdd(&counters[row], 1u);
  }
  __syncthreads();
  if (ticket != (unsigned)split - 1u) return;
  __threadfence();
  float acc = Op::identity();
  for (int k = threadIdx.x; k < split; k += 256) acc = Op::apply(acc, __ldcg(&partials[row * split + k]));
  acc = block_reduce<Op>(acc, slots[1]);
  if (threadIdx.x == 0) write_result<TO>(out, row, acc, scale, KIND);
}

constexpr int kColsVecCtasPerSm = 4;  // 60 registers (eight rows in flight per thread); a split launch is sized to exactly one wave of these

// How a reduction over a leading / middle axis is laid over the GPU (inner % 4 == 0).
struct ColPlan {
  int lanes;          // L: lanes per row, 4*L columns per CTA
  int64_t col_tiles;  // CTAs side by side along the inner axis
  int split;          // segments of the reduced axis
  int64_t seg;        // rows per segment (a multiple of 256/L)
  size_t counters_bytes, bytes;  // scratch: one counter per (outer, column tile), then split * 4*L partials for each
};

ColPlan col_plan(int64_t outer, int64_t n, int64_t inner, bool may_split) {
  ColPlan c;
  c.lanes = inner >= 128 ? 32 : inner >= 64 ? 16 : 8;
  const int64_t W = 4 * c.lanes, G = 256 / c.lanes;
  c.col_tiles = (inner + W - 1) / W;
  const int64_t base = outer * c.col_tiles, target = (int64_t)kSmCount * kColsVecCtasPerSm;
  int64_t split = may_split && base < target ? target / base : 1;  // rounded down: never a second, partly filled wave
  if (split > n / (4 * G)) split = n / (4 * G);  // at least four trips over the rows per segment
  if (split < 1) split = 1;
  c.seg = ((n + split - 1) / split + G - 1) / G * G;
  if (c.seg < G) c.seg = G;
  c.split = (int)((n + c.seg - 1) / c.seg);
  if (c.split < 1) c.split = 1;
  c.counters_bytes = c.split > 1 ? (((size_t)base * sizeof(unsigned)) + 255) & ~(size_t)255 : 0;
  c.bytes = c.split > 1 ? c.counters_bytes + (size_t)base * c.split * W * sizeof(float) : 0;
  return c;
}

template <typename T, typename TO, int KIND, int L>
__global__ void __launch_bounds__(256, kColsVecCtasPerSm) reduce_cols_vec(const T* __restrict__ x, TO* __restrict__ out, int64_t n, int64_t inner, int64_t col_tiles,
                                                       int split, int64_t seg, int64_t items, float scale, unsigned* __restrict__ counters,
                                                       float* __restrict__ partials) {
  using Op = typename KindOp<KIND>::Op;
  constexpr int G = 256 / L, W = 4 * L;
  __shared__ float tile[G][W];
  __shared__ unsigned ticket;
  const int tx = threadIdx.x % L, ty = threadIdx.x / L;
  for (int64_t item = blockIdx.x; item < items; item += gridDim.x) {
    const int part = (int)(item % split);
    const int64_t tile_id = item / split, ct = tile_id % col_tiles, o = tile_id / col_tiles;
    const int64_t c = ct * W + 4 * tx;
    const int64_t lo = (int64_t)part * seg, hi = lo + seg < n ? lo + seg : n;
    float acc[4][4];
#pragma unroll
    for (int u = 0; u < 4; ++u)
#pragma unroll
      for (int k = 0; k < 4; ++k) acc[u][k] = Op::identity();
    if (c < inner) {
      const T* p = x + o * n * inner + c;
      int64_t r = lo + ty;
      for (; r + 7 * G < hi; r += 8 * G) {  // eight rows in flight per thread
        float a[8][4];
#pragma unroll
        for (int u = 0; u < 8; ++u) load4<T>(p + (r + u * G) * inner, a[u]);
#pragma unroll
        for (int u = 0; u < 8; ++u)
#pragma unroll
          for (int k = 0; k < 4; ++k) acc[u & 3][k] = Op::apply(acc[u & 3][k], prep<KIND>(a[u][k]));
      }
      for (; r + 3 * G < hi; r += 4 * G) {  // four rows in flight per thread
        float a[4][4];
#pragma unroll
        for (int u = 0; u < 4; ++u) load4<T>(p + (r + u * G) * inner, a[u]);
#pragma unroll
        for (int u = 0; u < 4; ++u)
#pragma unroll
          for (int k = 0; k < 4; ++k) acc[u][k] = Op::apply(acc[u][k], prep<KIND>(a[u][k]));
      }
      for (; r < hi; r += G) {
        float a[4];
        load4<T>(p + r * inner, a);
#pragma unroll
        for (int k = 0; k < 4; ++k) acc[0][k] = Op::apply(acc[0][k], prep<KIND>(a[k]));
      }
    }
#pragma unroll
    for (int k = 0; k < 4; ++k) tile[ty][4 * tx + k] = Op::apply(Op::apply(acc[0][k], acc[1][k]), Op::apply(acc[2][k], acc[3][k]));
    __syncthreads();
    const bool owner = threadIdx.x < W && ct * W + threadIdx.x < inner;  // one thread per column of the tile
    float v = Op::identity();
    if (threadIdx.x < W) {
#pragma unroll 8
      for (int g = 0; g < G; ++g) v = Op::apply(v, tile[g][threadIdx.x]);
    }
    if (split == 1) {
      if (owner) write_result<TO>(out, o * inner + ct * W + threadIdx.x, v, scale, KIND);
    } else {
      if (threadIdx.x < W) {
        __stcg(&partials[item * W + threadIdx.x], v);
        __threadfence();  // the partials are visible before the ticket is
      }
      __syncthreads();
      if (threadIdx.x == 0) ticket = atomicAdd(&counters[tile_id], 1u);
      __syncthreads();
      if (ticket == (unsigned)split - 1u) {  // the last segment of this tile to finish folds them all, in order
        __threadfence();
        constexpr int kGroups = 256 / W;  // thread groups side by side over the partials: group g folds segments g, g + kGroups, ...
        const int col = threadIdx.x % W, grp = threadIdx.x / W;
        float a = Op::identity();
#pragma unroll 4
        for (int k = grp; k < split; k += kGroups) a = Op::apply(a, __ldcg(&partials[(tile_id * split + k) * W + col]));
        tile[grp][col] = a;  // every thread passed the barrier after the last read of tile
        __syncthreads();
        if (owner) {
          float r = tile[0][threadIdx.x];
#pragma unroll
          for (int g = 1; g < kGroups; ++g) r = Op::apply(r, tile[g][threadIdx.x]);
          write_result<TO>(out, o * inner + ct * W + threadIdx.x, r, scale, KIND);
        }
      }
    }
    __syncthreads();  // tile and ticket are reused by the next item
  }
}

template <typename T, typename TO, int KIND>
__global__ void __launch_bounds__(256) reduce_cols(const T* __restrict__ x, TO* __restrict__ out, int64_t outer,
                                                   int64_t n, int64_t inner, float scale) {
  using Op = typename KindOp<KIND>::Op;
  __shared__ float tile[8][33];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const int64_t tiles_per_outer = (inner + 31) / 32;
  const int64_t ntiles = outer * tiles_per_outer;
  for (int64_t t = blockIdx.x; t < ntiles; t += gridDim.x) {
    const int64_t o = t / tiles_per_outer, i = (t % tiles_per_outer) * 32 + tx;
    float acc = Op::identity();
    if (i < inner) {
      const T* p = x + o * n * inner + i;
      for (int64_t r = ty; r < n; r += 8) acc = Op::apply(acc, prep<KIND>(to_f32<T>(p[r * inner])));
    }
    tile[ty][tx] = acc;
    __syncthreads();
    if (ty == 0 && i < inner) {
#pragma unroll
      for (int k = 1; k < 8; ++k) acc = Op::apply(acc, tile[k][tx]);
      write_result<TO>(out, o * inner + i, acc, scale, KIND);
    }
    __syncthreads();
  }
}

template <typename T, typename TO, int KIND>
int run(const void* xv, void* outv, int64_t outer, int64_t n, int64_t inner, float scale, cudaStream_t s, void* scratch, size_t scratch_bytes) {
  const T* x = static_cast<const T*>(xv);
  TO* out = static_cast<TO*>(outv);
  if (inner == 1) {
    // 4-element vectors need every row start aligned to the vector's byte width: a base
    // pointer aligned to 16 bytes and n % 4 == 0 cover every T used here.
    const bool vec = aligned16(x) && n % 4 == 0;
    const int want = scratch && scratch_bytes >= kRowScratchBytes ? row_split_factor(outer, n, inner) : 1;
    if (want > 1) {
      int64_t seg = (n + want - 1) / want;
      seg = (seg + kSplitAlign - 1) / kSplitAlign * kSplitAlign;
      const int split = (int)((n + seg - 1) / seg);  // no empty segment
      unsigned* counters = static_cast<unsigned*>(scratch);
      float* partials = reinterpret_cast<float*>(counters + kSplitCounters);
      const int grid = (int)(outer * split);
      IB200_CUDA_OK(cudaMemsetAsync(counters, 0, (size_t)outer * sizeof(unsigned), s));  // the scratch area may hold anything
      if (vec) reduce_rows_split<T, TO, KIND, true><<<grid, 256, 0, s>>>(x, out, n, split, seg, scale, counters, partials);
      else reduce_rows_split<T, TO, KIND, false><<<grid, 256, 0, s>>>(x, out, n, split, seg, scale, counters, partials);
    } else if (vec && n <= 128 && outer >= 4096) {
      const int lanes = n <= 64 ? 8 : 16;
      const int64_t blocks = (outer + 256 / lanes - 1) / (256 / lanes);
      const int grid = (int)(blocks < (int64_t)kSmCount * 32 ? blocks : (int64_t)kSmCount * 32);
      if (lanes == 8) reduce_rows_sub<T, TO, KIND, 8><<<grid, 256, 0, s>>>(x, out, outer, (int)n, scale);
      else reduce_rows_sub<T, TO, KIND, 16><<<grid, 256, 0, s>>>(x, out, outer, (int)n, scale);
    } else if (n <= 2048) {
      const int64_t blocks = (outer + 7) / 8;
      const int grid = (int)(blocks < (int64_t)kSmCount * 16 ? blocks : (int64_t)kSmCount * 16);
      if (vec) reduce_rows_warp<T, TO, KIND, true><<<grid, 256, 0, s>>>(x, out, outer, n, scale);
      else reduce_rows_warp<T, TO, KIND, false><<<grid, 256, 0, s>>>(x, out, outer, n, scale);
    } else {
      const int grid = (int)(outer < (int64_t)kSmCount * 8 ? outer : (int64_t)kSmCount * 8);
      if (vec) reduce_rows_block<T, TO, KIND, true><<<grid, 256, 0, s>>>(x, out, outer, n, scale);
      else reduce_rows_block<T, TO, KIND, false><<<grid, 256, 0, s>>>(x, out, outer, n, scale);
    }
  } else if (aligned16(x) && inner % 4 == 0 && n >= 1) {
    ColPlan cp = col_plan(outer, n, inner, scratch != nullptr);
    if (cp.bytes > scratch_bytes) cp = col_plan(outer, n, inner, false);
    if (cp.split == 1 && outer * cp.col_tiles < 2 * (int64_t)kSmCount) {
      // too few wide tiles to fill the GPU and no scratch to split with: the narrow tiles give four times as many CTAs
      const int64_t tiles = outer * ((inner + 31) / 32);
      const int grid = (int)(tiles < (int64_t)kSmCount * 8 ? tiles : (int64_t)kSmCount * 8);
      reduce_cols<T, TO, KIND><<<grid, 256, 0, s>>>(x, out, outer, n, inner, scale);
      return cudaPeekAtLastError() == cudaSuccess ? IB200_OK : cuda_fail(cudaGetLastError(), "reduce launch");
    }
    unsigned* counters = static_cast<unsigned*>(scratch);
    float* partials = cp.split > 1 ? reinterpret_cast<float*>(static_cast<char*>(scratch) + cp.counters_bytes) : nullptr;
    if (cp.split > 1) IB200_CUDA_OK(cudaMemsetAsync(counters, 0, cp.counters_bytes, s));
    const int64_t items = outer * cp.col_tiles * cp.split;
    const int grid = (int)(items < (int64_t)kSmCount * 32 ? items : (int64_t)kSmCount * 32);
    if (cp.lanes == 32) reduce_cols_vec<T, TO, KIND, 32><<<grid, 256, 0, s>>>(x, out, n, inner, cp.col_tiles, cp.split, cp.seg, items, scale, counters, partials);
    else if (cp.lanes == 16) reduce_cols_vec<T, TO, KIND, 16><<<grid, 256, 0, s>>>(x, out, n, inner, cp.col_tiles, cp.split, cp.seg, items, scale, counters, partials);
    else reduce_cols_vec<T, TO, KIND, 8><<<grid, 256, 0, s>>>(x, out, n, inner, cp.col_tiles, cp.split, cp.seg, items, scale, counters, partials);
  } else {
    const int64_t tiles = outer * ((inner + 31) / 32);
    const int grid = (int)(tiles < (int64_t)kSmCount * 8 ? tiles : (int64_t)kSmCount * 8);
    reduce_cols<T, TO, KIND><<<grid, 256, 0, s>>>(x, out, outer, n, inner, scale);
  }
  return cudaPeekAtLastError() == cudaSuccess ? IB200_OK : cuda_fail(cudaGetLastError(), "reduce launch");
}

template <typename T, int KIND> int pick_out(const void* x, void* out, int out_dtype, int64_t outer, int64_t n,
                                             int64_t inner, float scale, cudaStream_t s, void* scratch, size_t scratch_bytes) {
  if (KIND == IB200_REDUCE_ANY) {
    if (out_dtype != IB200_BOOL && out_dtype != IB200_U8) return fail(IB200_ERR_INVALID, "reduce_any writes one byte per result: out_dtype must be bool");
    return run<T, uint8_t, KIND>(x, out, outer, n, inner, scale, s, scratch, scratch_bytes);
  }
  switch (out_dtype) {
    case IB200_F32: return run<T, float, KIND>(x, out, outer, n, inner, scale, s, scratch, scratch_bytes);
    case IB200_BF16: return run<T, __nv_bfloat16, KIND>(x, out, outer, n, inner, scale, s, scratch, scratch_bytes);
    case IB200_F16: return run<T, __half, KIND>(x, out, outer, n, inner, scale, s, scratch, scratch_bytes);
    default: return fail(IB200_ERR_UNSUPPORTED, "reduce: output dtype must be f32, bf16 or f16");
  }
}

template <int KIND> int pick_in(const void* x, void* out, int x_dtype, int out_dtype, int64_t outer, int64_t n,
                                int64_t inner, float scale, cudaStream_t s, void* scratch, size_t scratch_bytes) {
  switch (x_dtype) {
    case IB200_F32: return pick_out<float, KIND>(x, out, out_dtype, outer, n, inner, scale, s, scratch, scratch_bytes);
    case IB200_BF16: return pick_out<__nv_bfloat16, KIND>(x, out, out_dtype, outer, n, inner, scale, s, scratch, scratch_bytes);
    case IB200_F16: return pick_out<__half, KIND>(x, out, out_dtype, outer, n, inner, scale, s, scratch, scratch_bytes);
    case IB200_BOOL: case IB200_U8:
      if (KIND == IB200_REDUCE_ANY) return pick_out<uint8_t, KIND>(x, out, out_dtype, outer, n, inner, scale, s, scratch, scratch_bytes);
      return fail(IB200_ERR_UNSUPPORTED, "reduce: sum/max over a bool tensor is not covered");
    default: return fail(IB200_ERR_UNSUPPORTED, "reduce: input dtype must be f32, bf16, f16 or bool");
  }
}

}  // namespace

// Splitting pays when the rows alone cannot fill the GPU (fewer than two per SM) and each is long
// enough for several segments of at least 16 Ki elements; the aim is about four CTAs per SM.
namespace {
int row_split_factor(int64_t outer, int64_t reduce, int64_t inner) {
  if (inner != 1 || outer < 1 || outer >= 2 * kSmCount || outer > kSplitCounters || reduce < 65536) return 1;
  int64_t split = (4 * (int64_t)kSmCount + outer - 1) / outer;
  if (split > reduce / 16384) split = reduce / 16384;
  if (outer * split > kSplitPartials) split = kSplitPartials / outer;
  return split < 2 ? 1 : (int)split;
}
}  // namespace

size_t reduce_scratch_bytes(int64_t outer, int64_t reduce, int64_t inner) {
  if (outer < 1 || reduce < 1 || inner < 1) return 0;
  if (inner == 1) return row_split_factor(outer, reduce, inner) > 1 ? kRowScratchBytes : 0;
  return inner % 4 == 0 ? col_plan(outer, reduce, inner, true).bytes : 0;
}

int launch_reduce(const void* x, void* out, int x_dtype, int out_dtype, int kind, int64_t outer, int64_t reduce,
                  int64_t inner, float scale, cudaStream_t s, void* scratch, size_t scratch_bytes) {
  if (outer < 0 || reduce < 0 || inner < 0) return fail(IB200_ERR_INVALID, "reduce: negative extent");
  if (outer == 0 || inner == 0) return IB200_OK;  // empty result
  if (beyond_any_device(outer, reduce > 0 ? reduce : 1, inner)) return fail(IB200_ERR_INVALID, "reduce: more than 2^40 elements");
  if (!out || (!x && reduce > 0)) return fail(IB200_ERR_INVALID, "reduce: null pointer");
  if (reduce == 0 && kind == IB200_REDUCE_MAX) return fail(IB200_ERR_INVALID, "reduce_max over an empty axis has no identity");
  switch (kind) {
    case IB200_REDUCE_SUM: return pick_in<IB200_REDUCE_SUM>(x, out, x_dtype, out_dtype, outer, reduce, inner, scale, s, scratch, scratch_bytes);
    case IB200_REDUCE_MAX: return pick_in<IB200_REDUCE_MAX>(x, out, x_dtype, out_dtype, outer, reduce, inner, scale, s, scratch, scratch_bytes);
    case IB200_REDUCE_ANY: return pick_in<IB200_REDUCE_ANY>(x, out, x_dtype, out_dtype, outer, reduce, inner, scale, s, scratch, scratch_bytes);
    default: return fail(IB200_ERR_INVALID, "reduce: unknown kind");
  }
}

}  // namespace ib200
