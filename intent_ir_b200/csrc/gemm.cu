// C[M,N] = act(A[M,K] · B + bias), fp32 accumulation.
//
// Tensor-core path (bf16 or f16 operands, and f32 operands as TF32 when the caller allows it; K and
// N multiples of 8).  Two persistent, warp-specialised sm_100a kernels share the roles below:
// large products run on PAIRS of CTAs that share 256 x 256 output tiles (tcgen05 cta_group::2,
// described further down), everything else on one CTA per SM with 128 x BN output tiles (BN =
// 256, 192 or 128, chosen per problem to waste the fewest SM-waves).  K advances in blocks of
// 128 bytes (64 16-bit or 32 32-bit elements):
//   warp 0   : TMA producer — cp.async.bulk.tensor (128-byte swizzle) into a 4..6-stage
//              shared-memory ring, completion on mbarriers;
//   warp 1   : allocates tensor memory and issues tcgen05.mma (cta_group::1, kind::f16 with
//              M=128 N=BN K=16, or kind::tf32 with K=8) from one elected thread; tcgen05.commit releases ring
//              stages back to the producer and publishes finished accumulators;
//   warps 2-5: epilogue — tcgen05.ld of the fp32 accumulator (one row per thread), + bias,
//              activation, conversion, 16-byte stores.
// Two accumulators of up to 256 columns share the 512 TMEM columns, so the epilogue of tile i overlaps
// the main loop of tile i+1.  A is K-major; 16-bit B is read as stored: [K,N] row-major is the
// MN-major operand form (the descriptor's major bit), [N,K] (transpose_b) is K-major — no
// transposition pass either way.  A 32-bit (TF32) B is taken K-major only: a [K,N] one is
// first transposed into scratch (the MN-major form of 32-bit operands wants a shared-memory
// layout this kernel does not produce).  Every mbarrier wait is bounded: on expiry the thread
// records where it gave up in *status and the kernel drains and exits, so a wrong
// descriptor can produce a wrong answer or an error code, never a hung GPU.
//
// Tail split: tiles are handed out round by round to the resident CTAs, and a last round that
// fills less than half of them would leave most SMs idle for a whole tile time (4096^3: 512
// tiles on 148 SMs = 3.46 rounds).  With scratch memory, every tile of that last round is cut
// along K into `split` slices, one work unit each; a unit stores its fp32 partial tile to
// scratch, fences and draws a ticket per 32-row band, and the epilogue warp that draws the
// last ticket sums the slices in slice order (the same order on every run) and applies bias
// and activation.  Nobody waits for anybody.
//
// Replaces the reference's opt-in TF32 wmma/mma.sync kernel (kernels/wmma_matmul.cuh) and
// its FMA default (kernels/matmul_fallback.cuh); the bias+activation epilogue that the
// reference leaves as separate ops (pipeline/tilelang/core.py:895-901) is fused.
//
// FMA path: every other shape / dtype (fp32 operands, ragged K or N): 64x64 tiles, 4x4 per
// thread, operands staged through shared memory.
#include <cuda.h>

#include <cstdlib>

#include "common.cuh"

namespace ib200 {
namespace {

// ============================== tcgen05 path ==========================================
constexpr int BM = 128;
constexpr int KROW_BYTES = 128;                    // one K block = one 128-byte swizzled row per tile row
constexpr int A_STAGE_BYTES = BM * KROW_BYTES;     // 16 KiB
// operand kinds: element size, elements per K block, K extent of one MMA, instruction-descriptor format code
enum { KIND_BF16 = 0, KIND_F16 = 1, KIND_TF32 = 2 };
template <int KIND> struct KindCfg {
  static constexpr int ESZ = KIND == KIND_TF32 ? 4 : 2;
  static constexpr int BK = KROW_BYTES / ESZ;       // 64 or 32 elements
  static constexpr int UMMA_K = 32 / ESZ;           // 16 or 8 elements = 32 bytes of every row per MMA
  static constexpr uint32_t FMT = KIND == KIND_BF16 ? 1u : KIND == KIND_F16 ? 0u : 2u;
};
// The N extent of a tile is a template parameter (256, 192 or 128): the launcher picks the one
// that minimises waves x time-per-tile for the problem at hand (narrow N, ragged tile counts).
template <int BN> struct TileCfg {
  static constexpr int B_STAGE_BYTES = KROW_BYTES * BN;
  static constexpr int STAGE_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;      // 48 / 40 / 32 KiB, multiples of 1 KiB
  static constexpr int STAGES = BN == 256 ? 4 : (BN == 192 ? 5 : 6);     // 192 / 200 / 192 KiB of ring
  static constexpr int SMEM = STAGES * STAGE_BYTES + 1024 /*alignment slack*/ + 256 /*barriers*/;
};
constexpr int kMaxSplit = 4;  // K slices per tail tile, at most
constexpr int ACC_COLS = 256;  // TMEM columns reserved per accumulator buffer (two buffers = all 512)
constexpr int GEMM_THREADS = 192;
constexpr uint64_t WAIT_LIMIT_NS = 2000000000ull;   // 2 s per wait, then give up

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ uint64_t now_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
      : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
  return ok != 0;
}
// Bounded wait.  Returns false (after recording `code`) when the limit expires or when
// another thread has already flagged a failure.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int32_t* status, int code) {
  if (mbar_try(bar, parity)) return true;
  const uint64_t t0 = now_ns();
  uint32_t spins = 0;
  while (!mbar_try(bar, parity)) {
    if ((++spins & 0x3ff) == 0) {
      if (*abort_flag) return false;
      if (now_ns() - t0 > WAIT_LIMIT_NS) {
        *abort_flag = 1;
        if (status) atomicCAS(status, 0, code);
        return false;
      }
    }
  }
  return true;
}

__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1) : "memory");
}

// 64-bit shared-memory matrix descriptor (tcgen05): start address, leading / stride byte
// offsets (all >> 4), descriptor version 1, 128-byte swizzle.
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFF) >> 4);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32;
  d |= (uint64_t)1 << 46;  // descriptor version (Blackwell)
  d |= (uint64_t)2 << 61;  // SWIZZLE_128B
  return d;
}

template <int KIND>
__device__ __forceinline__ void umma(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  if (KIND == KIND_TF32) {
    asm volatile(
        "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
        " tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
  } else {
    asm volatile(
        "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
        " tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
  }
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr) : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

struct GemmParams {
  int M, N, K;
  int b_kmajor;  // 1: B is [N,K] (transpose_b)
  int act;
  const void* bias;
  void* c;
  int32_t* status;
  // work units: tiles [0, full_tiles) whole, every later tile as `split` K slices (split == 1: no tail split)
  int full_tiles, split;
  int* tickets;     // [split tiles][4 row bands], zero before the launch, left zero by it
  float* partial;   // [split tiles][split][BM][BN] fp32
  // CTA pairs: tiles [0, narrow_from) whole, every later tile as two units of half the width (== tiles: none)
  int narrow_from;
};

struct Unit {
  int tile, kb0, kb1, slice;  // slice < 0: a whole tile
};
__device__ __forceinline__ Unit decode_unit(int u, const GemmParams& p, int kblocks) {
  Unit w;
  if (u < p.full_tiles) {
    w.tile = u; w.kb0 = 0; w.kb1 = kblocks; w.slice = -1;
  } else {
    const int idx = u - p.full_tiles, per = (kblocks + p.split - 1) / p.split;
    w.tile = p.full_tiles + idx / p.split;
    w.slice = idx % p.split;
    w.kb0 = w.slice * per;
    w.kb1 = w.kb0 + per < kblocks ? w.kb0 + per : kblocks;
  }
  return w;
}

template <typename TOut> __device__ __forceinline__ uint32_t pack2(float a, float b);
template <> __device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float a, float b) {
  __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}
template <> __device__ __forceinline__ uint32_t pack2<__half>(float a, float b) {
  __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}
template <> __device__ __forceinline__ uint32_t pack2<float>(float a, float) { return __float_as_uint(a); }

// bias, activation, conversion and 16-byte stores for 8 consecutive columns of one row
template <typename TOut>
__device__ __forceinline__ void finish8(float (&v)[8], const TOut* bias, int col, int act, TOut* crow) {
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    if (bias) v[j] += to_f32<TOut>(bias[col + j]);
    if (act == IB200_ACT_RELU) v[j] = max_nan(v[j], 0.0f);
  }
  if (sizeof(TOut) == 2) {
    uint4 q;
    q.x = pack2<TOut>(v[0], v[1]); q.y = pack2<TOut>(v[2], v[3]); q.z = pack2<TOut>(v[4], v[5]); q.w = pack2<TOut>(v[6], v[7]);
    *reinterpret_cast<uint4*>(crow + col) = q;
  } else {
    *reinterpret_cast<float4*>(crow + col) = make_float4(v[0], v[1], v[2], v[3]);
    *reinterpret_cast<float4*>(crow + col + 4) = make_float4(v[4], v[5], v[6], v[7]);
  }
}

template <typename TOut, int BN, int KIND>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const GemmParams p) {
  constexpr int STAGES = TileCfg<BN>::STAGES, STAGE_BYTES = TileCfg<BN>::STAGE_BYTES;
  constexpr int BK = KindCfg<KIND>::BK, UMMA_K = KindCfg<KIND>::UMMA_K, NBOX = KROW_BYTES / KindCfg<KIND>::ESZ;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
  uint64_t* empty = full + STAGES;
  uint64_t* acc_full = empty + STAGES;
  uint64_t* acc_empty = acc_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_m = (p.M + BM - 1) / BM, tiles_n = (p.N + BN - 1) / BN;
  const int ntiles = tiles_m * tiles_n;
  const int kblocks = (p.K + BK - 1) / BK;
  const int nunits = p.full_tiles + (ntiles - p.full_tiles) * p.split;

  if (threadIdx.x == 0) {
    for (int i = 0; i < STAGES; ++i) { mbar_init(&full[i], 1); mbar_init(&empty[i], 1); }
    for (int i = 0; i < 2; ++i) { mbar_init(&acc_full[i], 1); mbar_init(&acc_empty[i], 4); }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {  // allocate all 512 TMEM columns (one CTA per SM owns the whole tensor memory)
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(512) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------------
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int u = blockIdx.x; u < nunits && ok; u += gridDim.x) {
        const Unit w = decode_unit(u, p, kblocks);
        const int m0 = (w.tile / tiles_n) * BM, n0 = (w.tile % tiles_n) * BN;
        for (int kb = w.kb0; kb < w.kb1; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!(ok = mbar_wait(&empty[s], ph ^ 1, abort_flag, p.status, 1))) break;
          uint8_t* sa = smem + s * STAGE_BYTES;
          uint8_t* sb = sa + A_STAGE_BYTES;
          mbar_expect_tx(&full[s], STAGE_BYTES);
          tma_load_2d(sa, &map_a, &full[s], kb * BK, m0);
          if (p.b_kmajor) {
            tma_load_2d(sb, &map_b, &full[s], kb * BK, n0);  // one box: BK (K) x BN (N rows)
          } else {
#pragma unroll
            for (int j = 0; j < BN / NBOX; ++j)  // boxes of NBOX (N, 128 bytes) x BK (K rows)
              tma_load_2d(sb + j * (BK * KROW_BYTES), &map_b, &full[s], n0 + j * NBOX, kb * BK);
          }
        }
      }
      // drain: every stage that was armed must land before the CTA may exit
      for (int i = 0; i < STAGES; ++i) {
        if (it == 0) break;
        const uint32_t last = it - 1;  // the newest armed iteration
        const int s = i;
        // the newest iteration that used stage s
        if (last < (uint32_t)s) continue;
        const uint32_t j = last - ((last - s) % STAGES);
        (void)mbar_wait(&full[s], (j / STAGES) & 1, abort_flag, nullptr, 0);
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ---------------------------------------
    if (lane == 0) {
      const uint32_t idesc = (1u << 4) | (KindCfg<KIND>::FMT << 7) | (KindCfg<KIND>::FMT << 10) | ((p.b_kmajor ? 0u : 1u) << 16) |
                             ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
      uint32_t it = 0, t_local = 0;
      bool ok = true;
      for (int u = blockIdx.x; u < nunits && ok; u += gridDim.x, ++t_local) {
        const Unit w = decode_unit(u, p, kblocks);
        const int buf = t_local & 1;
        const uint32_t acc_ph = (t_local >> 1) & 1;
        if (!(ok = mbar_wait(&acc_empty[buf], acc_ph ^ 1, abort_flag, p.status, 2))) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + buf * ACC_COLS;
        for (int kb = w.kb0; kb < w.kb1; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!(ok = mbar_wait(&full[s], ph, abort_flag, p.status, 3))) break;
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + s * STAGE_BYTES), sb = sa + A_STAGE_BYTES;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            // A: K-major, 128-byte swizzled rows; one MMA's K extent = 32 bytes inside the row
            const uint64_t adesc = umma_desc(sa + k * 32, 16, 1024);
            // B: K-major ([N,K]) like A, or MN-major ([K,N]): 128-byte column chunks BK*128 bytes
            // apart (leading offset), 8-row K groups 1024 bytes apart (stride offset); one
            // MMA's K extent = UMMA_K rows of 128 bytes
            const uint64_t bdesc = p.b_kmajor ? umma_desc(sb + k * 32, 16, 1024)
                                              : umma_desc(sb + k * (UMMA_K * KROW_BYTES), BK * KROW_BYTES, 1024);
            umma<KIND>(d_tmem, adesc, bdesc, idesc, (kb != w.kb0 || k != 0) ? 1u : 0u);
          }
          umma_commit(&empty[s]);  // stage reusable once these MMAs have read it
        }
        if (ok) umma_commit(&acc_full[buf]);
      }
    }
  } else {
    // ------------------------------ epilogue (warps 2..5) ----------------------------
    const int quarter = warp & 3;  // TMEM lanes 32*quarter .. +31 are this warp's
    uint32_t t_local = 0;
    bool ok = true;
    for (int u = blockIdx.x; u < nunits && ok; u += gridDim.x, ++t_local) {
      const Unit w = decode_unit(u, p, kblocks);
      const int buf = t_local & 1;
      const uint32_t acc_ph = (t_local >> 1) & 1;
      const int m0 = (w.tile / tiles_n) * BM, n0 = (w.tile % tiles_n) * BN;
      ok = mbar_wait(&acc_full[buf], acc_ph, abort_flag, p.status, 4);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      const int row = m0 + quarter * 32 + lane;
      TOut* crow = static_cast<TOut*>(p.c) + (size_t)row * p.N;
      const TOut* bias = static_cast<const TOut*>(p.bias);
      const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + buf * ACC_COLS;
      if (w.slice < 0) {
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          uint32_t r[32];
          tmem_ld32(taddr + c * 32, r);
          const int col0 = n0 + c * 32;
          if (row < p.M) {
#pragma unroll
            for (int g = 0; g < 32; g += 8) {
              const int col = col0 + g;
              if (col >= p.N) break;  // N % 8 == 0: a group of 8 columns is all in or all out
              float v[8];
#pragma unroll
              for (int j = 0; j < 8; ++j) v[j] = __uint_as_float(r[g + j]);
              finish8<TOut>(v, bias, col, p.act, crow);
            }
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&acc_empty[buf]);
      } else {
        // a K slice of a tail tile: park the fp32 partial, then whoever parks last for this 32-row band adds
        // the slices up in slice order.  Parked layout per (tile, slice): [32-column chunk][4-column group][row][4],
        // so that the 32 rows of a warp write, and later read, 512 contiguous bytes per instruction.
        const int st = w.tile - p.full_tiles;
        const int trow = quarter * 32 + lane;
        float* mine = p.partial + (size_t)(st * p.split + w.slice) * BM * BN;
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          uint32_t r[32];
          tmem_ld32(taddr + c * 32, r);
#pragma unroll
          for (int g = 0; g < 8; ++g)
            __stcg(reinterpret_cast<float4*>(mine + ((size_t)(c * 8 + g) * BM + trow) * 4),
                   make_float4(__uint_as_float(r[4 * g]), __uint_as_float(r[4 * g + 1]), __uint_as_float(r[4 * g + 2]), __uint_as_float(r[4 * g + 3])));
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&acc_empty[buf]);  // the accumulator is free: the next unit's main loop may start
        __threadfence();
        __syncwarp();
        int ticket = 0;
        if (lane == 0) ticket = atomicAdd(&p.tickets[st * 4 + quarter], 1);
        ticket = __shfl_sync(0xffffffffu, ticket, 0);
        if (ticket == p.split - 1) {
          __threadfence();
          if (lane == 0) p.tickets[st * 4 + quarter] = 0;  // ready for the next launch
          const float* base = p.partial + (size_t)(st * p.split) * BM * BN;
#pragma unroll 1
          for (int c = 0; c < BN / 32; ++c) {
            const int col0 = n0 + c * 32;
            if (col0 >= p.N) break;
            float4 q[kMaxSplit][8];
#pragma unroll
            for (int sl = 0; sl < kMaxSplit; ++sl)  // every load of the chunk in flight before the first add
              if (sl < p.split) {
#pragma unroll
                for (int g = 0; g < 8; ++g)
                  q[sl][g] = __ldcg(reinterpret_cast<const float4*>(base + (size_t)sl * BM * BN + ((size_t)(c * 8 + g) * BM + trow) * 4));
              }
            if (row < p.M) {
#pragma unroll
              for (int g8 = 0; g8 < 4; ++g8) {
                const int col = col0 + g8 * 8;
                if (col >= p.N) break;
                float v[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
                for (int sl = 0; sl < kMaxSplit; ++sl)
                  if (sl < p.split) {
                    const float4 lo = q[sl][2 * g8], hi = q[sl][2 * g8 + 1];
                    v[0] += lo.x; v[1] += lo.y; v[2] += lo.z; v[3] += lo.w; v[4] += hi.x; v[5] += hi.y; v[6] += hi.z; v[7] += hi.w;
                  }
                finish8<TOut>(v, bias, col, p.act, crow);
              }
            }
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512) : "memory");
  }
}

// ============================== CTA pairs (cta_group::2) ==============================
// Two CTAs of a cluster share one 256 x BN output tile: CTA r of the pair stages rows
// r*128 .. +127 of A and columns r*(BN/2) .. of B, half of what a lone CTA stages for the same
// 128 x BN of output, and one tcgen05.mma.cta_group::2 issued by CTA 0 multiplies both
// halves: each SM's tensor core reads its own A rows and both halves of B, and leaves its
// 128 x BN block of the result in its own tensor memory.  Per CTA and K block the ring takes
// 16 KiB of A and BN/2 columns of B instead of BN, which is where the main loop of the
// one-CTA kernel spends its time (operand traffic into shared memory).
//
// Synchronisation, every wait on a barrier of the waiting CTA's own shared memory:
//   full[s]        in CTA 0 only: the operands of BOTH CTAs for stage s have landed — CTA 1's
//                  loads (cp.async.bulk.tensor with .cta_group::2) report their bytes to CTA 0's
//                  barrier, which expects two stages' worth;
//   empty[s]       per CTA: the MMAs that read the stage have completed — one tcgen05.commit in
//                  CTA 0 arrives on the barrier of both CTAs;
//   acc_full[b]    per CTA: accumulator b complete (the same kind of commit);
//   acc_empty[b]   in CTA 0, eight arrivals: the four epilogue warps of either CTA (CTA 1's
//                  arrive remotely).
// No load is multicast (each CTA loads only what it stages itself); every wait is bounded as in
// the one-CTA kernel, and both CTAs meet at a cluster barrier before either frees its tensor
// memory or exits.  (A first version passed the stage hand-offs between the CTAs through relay
// threads and remote arrives only; with two extra hops per stage the six-stage ring no longer
// covered the refill latency and it ran at half the speed of the one-CTA kernel.)
__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t map_to_cta(const void* local, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_u32(local)), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_remote(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// a tile into this CTA's shared memory whose bytes are counted on a barrier of either CTA of the pair
__device__ __forceinline__ void tma_load_2d_pair(void* dst, const CUtensorMap* map, uint32_t bar_cluster_addr, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes.cta_group::2 [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(dst)), "l"(map), "r"(bar_cluster_addr), "r"(c0), "r"(c1) : "memory");
}
template <int KIND>
__device__ __forceinline__ void umma_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  if (KIND == KIND_TF32) {
    asm volatile(
        "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
        " tcgen05.mma.cta_group::2.kind::tf32 [%0], %1, %2, %3, p;\n}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
  } else {
    asm volatile(
        "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
        " tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
  }
}
// completion of the MMAs issued so far, signalled to the barrier at this offset in BOTH CTAs of the pair
__device__ __forceinline__ void umma_commit_both(uint64_t* bar) {
  const uint16_t both = 3;
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(smem_u32(bar)), "h"(both) : "memory");
}

// Work units of the pair kernel.  On request (IB200_GEMM_NARROW_TAIL) the tiles of a last round that would occupy at
// most half of the pairs run as two units of half the width each (256 x 128), so that twice as many pairs share the
// round, with no partial sums to exchange.  4096^3: 256 tiles on 74 pairs are 3 full rounds and 34 tiles, i.e. 68
// narrow units.  Off by default: measured on 4096^3 bf16 it changes nothing (101.3 against 101.0 us, alternating
// runs) -- at the board's power cap the time of a product follows the energy it takes, not how evenly the SMs finish,
// and narrow units move more operand bytes per flop.  4096 x 5120 x 2048: 70.8 against 73.4 us.
struct PairUnit {
  int m_tile, n0, bn;
};
__device__ __forceinline__ PairUnit pair_unit(int u, int narrow_from, int tiles_n, int bn_wide) {
  PairUnit w;
  if (u < narrow_from) {
    w.m_tile = u / tiles_n;
    w.n0 = (u % tiles_n) * bn_wide;
    w.bn = bn_wide;
  } else {
    const int t = narrow_from + ((u - narrow_from) >> 1);
    w.m_tile = t / tiles_n;
    w.bn = bn_wide / 2;
    w.n0 = (t % tiles_n) * bn_wide + ((u - narrow_from) & 1) * w.bn;
  }
  return w;
}

template <int BN> struct PairCfg {
  static constexpr int B_STAGE_BYTES = KROW_BYTES * (BN / 2);
  static constexpr int STAGE_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;   // 32 KiB at BN = 256
  static constexpr int STAGES = BN == 256 ? 6 : 8;
  static constexpr int SMEM = STAGES * STAGE_BYTES + 1024 + 512;
};

template <typename TOut, int BN, int KIND>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(GEMM_THREADS, 1)
gemm_tcgen05_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                         const __grid_constant__ CUtensorMap map_b_narrow, const GemmParams p) {
  constexpr int STAGES = PairCfg<BN>::STAGES, STAGE_BYTES = PairCfg<BN>::STAGE_BYTES;
  constexpr int BK = KindCfg<KIND>::BK, UMMA_K = KindCfg<KIND>::UMMA_K, NBOX = KROW_BYTES / KindCfg<KIND>::ESZ;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
  uint64_t* empty = full + STAGES;
  uint64_t* acc_full = empty + STAGES;
  uint64_t* acc_empty = acc_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_rank();
  const int pair = blockIdx.x >> 1, npairs = gridDim.x >> 1;
  const int tiles_m = (p.M + 2 * BM - 1) / (2 * BM), tiles_n = (p.N + BN - 1) / BN;
  const int ntiles = tiles_m * tiles_n;
  const int nunits = p.narrow_from + 2 * (ntiles - p.narrow_from);  // tiles from narrow_from on run as two half-width units
  const int kblocks = (p.K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int i = 0; i < STAGES; ++i) { mbar_init(&full[i], 1); mbar_init(&empty[i], 1); }
    for (int i = 0; i < 2; ++i) { mbar_init(&acc_full[i], 1); mbar_init(&acc_empty[i], 8); }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {  // both CTAs of the pair allocate all 512 columns of their tensor memory
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(512) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // both CTAs run and have initialised their barriers: signals may cross from here on
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------ TMA producer (both CTAs) -------------------------
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int u = pair; u < nunits && ok; u += npairs) {
        const PairUnit w = pair_unit(u, p.narrow_from, tiles_n, BN);
        const int m0 = w.m_tile * (2 * BM) + (int)rank * BM, n0 = w.n0 + (int)rank * (w.bn / 2);
        const uint32_t stage_tx = 2 * (A_STAGE_BYTES + (w.bn / 2) * KROW_BYTES);
        for (int kb = 0; kb < kblocks; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!(ok = mbar_wait(&empty[s], ph ^ 1, abort_flag, p.status, 1))) break;
          uint8_t* sa = smem + s * STAGE_BYTES;
          uint8_t* sb = sa + A_STAGE_BYTES;
          const uint32_t bar = map_to_cta(&full[s], 0);  // CTA 0's barrier counts the bytes of both CTAs
          if (rank == 0) mbar_expect_tx(&full[s], stage_tx);
          tma_load_2d_pair(sa, &map_a, bar, kb * BK, m0);
          if (p.b_kmajor) {
            tma_load_2d_pair(sb, w.bn == BN ? &map_b : &map_b_narrow, bar, kb * BK, n0);  // one box: BK (K) x this CTA's N rows
          } else {
            for (int j = 0; j < (w.bn / 2) / NBOX; ++j)
              tma_load_2d_pair(sb + j * (BK * KROW_BYTES), &map_b, bar, n0 + j * NBOX, kb * BK);
          }
        }
      }
      if (rank == 0) {  // drain: every armed stage lands (in both CTAs) before the pair may leave
        for (int i = 0; i < STAGES; ++i) {
          if (it == 0) break;
          const uint32_t last = it - 1;
          if (last < (uint32_t)i) continue;
          const uint32_t j = last - ((last - i) % STAGES);
          (void)mbar_wait(&full[i], (j / STAGES) & 1, abort_flag, nullptr, 0);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && rank == 0) {
      // ------------------------------ MMA issuer (CTA 0) -------------------------------
      const uint32_t idesc_wide = (1u << 4) | (KindCfg<KIND>::FMT << 7) | (KindCfg<KIND>::FMT << 10) | ((p.b_kmajor ? 0u : 1u) << 16) |
                                  ((uint32_t)(BN >> 3) << 17) | ((uint32_t)((2 * BM) >> 4) << 24);
      const uint32_t idesc_narrow = (idesc_wide & ~(0x3Fu << 17)) | ((uint32_t)((BN / 2) >> 3) << 17);
      uint32_t it = 0, t_local = 0;
      bool ok = true;
      for (int u = pair; u < nunits && ok; u += npairs, ++t_local) {
        const uint32_t idesc = u < p.narrow_from ? idesc_wide : idesc_narrow;
        const int buf = t_local & 1;
        const uint32_t acc_ph = (t_local >> 1) & 1;
        if (!(ok = mbar_wait(&acc_empty[buf], acc_ph ^ 1, abort_flag, p.status, 2))) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + buf * ACC_COLS;
        for (int kb = 0; kb < kblocks; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!(ok = mbar_wait(&full[s], ph, abort_flag, p.status, 3))) break;
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + s * STAGE_BYTES), sb = sa + A_STAGE_BYTES;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            const uint64_t adesc = umma_desc(sa + k * 32, 16, 1024);
            const uint64_t bdesc = p.b_kmajor ? umma_desc(sb + k * 32, 16, 1024)
                                              : umma_desc(sb + k * (UMMA_K * KROW_BYTES), BK * KROW_BYTES, 1024);
            umma_pair<KIND>(d_tmem, adesc, bdesc, idesc, (kb != 0 || k != 0) ? 1u : 0u);
          }
          umma_commit_both(&empty[s]);
        }
        if (ok) umma_commit_both(&acc_full[buf]);
      }
    }
  } else {
    // ------------------------------ epilogue (warps 2..5, both CTAs) -------------------
    const int quarter = warp & 3;
    uint32_t t_local = 0;
    bool ok = true;
    for (int u = pair; u < nunits && ok; u += npairs, ++t_local) {
      const PairUnit w = pair_unit(u, p.narrow_from, tiles_n, BN);
      const int buf = t_local & 1;
      const uint32_t acc_ph = (t_local >> 1) & 1;
      const int m0 = w.m_tile * (2 * BM) + (int)rank * BM, n0 = w.n0;
      ok = mbar_wait(&acc_full[buf], acc_ph, abort_flag, p.status, 4);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      const int row = m0 + quarter * 32 + lane;
      TOut* crow = static_cast<TOut*>(p.c) + (size_t)row * p.N;
      const TOut* bias = static_cast<const TOut*>(p.bias);
      const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + buf * ACC_COLS;
#pragma unroll 1
      for (int c = 0; c < w.bn / 32; ++c) {
        uint32_t r[32];
        tmem_ld32(taddr + c * 32, r);
        const int col0 = n0 + c * 32;
        if (row < p.M) {
#pragma unroll
          for (int g = 0; g < 32; g += 8) {
            const int col = col0 + g;
            if (col >= p.N) break;
            float v[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) v[j] = __uint_as_float(r[g + j]);
            finish8<TOut>(v, bias, col, p.act, crow);
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        if (rank == 0) mbar_arrive(&acc_empty[buf]);
        else mbar_arrive_remote(map_to_cta(&acc_empty[buf], 0));
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // nobody frees tensor memory or leaves while the other CTA may still signal it or read its shared memory
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512) : "memory");
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

int get_encoder(EncodeTiledFn* out) {
  static EncodeTiledFn cached = nullptr;
  if (!cached) {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    IB200_CUDA_OK(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q));
    if (q != cudaDriverEntryPointSuccess || !fn) return fail(IB200_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    cached = reinterpret_cast<EncodeTiledFn>(fn);
  }
  *out = cached;
  return IB200_OK;
}

// row-major [rows, cols] tensor of 2- or 4-byte elements, box [box_rows, box_cols], 128-byte swizzle
int make_map(EncodeTiledFn enc, CUtensorMap* map, const void* base, int kind, int64_t rows, int64_t cols, int box_rows, int box_cols) {
  const int esz = kind == KIND_TF32 ? 4 : 2;
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)cols * esz};
  cuuint32_t box[2] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  const CUtensorMapDataType dt = kind == KIND_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                 : kind == KIND_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
  CUresult r = enc(map, dt, 2, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(IB200_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult " + std::to_string((int)r));
  return IB200_OK;
}

// How the tiles of a problem are handed out: `full` tiles whole, the rest as `split` K slices each.
struct SplitPlan {
  int bn, full_tiles, split;
  int64_t tiles;
  double cost;  // rounds of the resident CTAs, in units of one 256-wide tile
  size_t scratch;
};
// a slice shorter than this many K blocks costs more in the exchange of partial tiles (a fixed 5-8 us) than the
// idle SMs it saves: measured on 2560 x 2560 x 1024 (16 blocks, two slices), 27.9 us split against 19.9 us whole
constexpr int kMinSliceBlocks = 16;

SplitPlan split_plan(int bn, int64_t m, int64_t n, int64_t kblocks, bool allow_split) {
  static const double penalty[3] = {1.0, 1.18, 1.58};  // time per output column, measured on 4096^3 (256 / 192 / 128 wide)
  SplitPlan sp{};
  sp.bn = bn;
  sp.tiles = ((m + BM - 1) / BM) * ((n + bn - 1) / bn);
  const int64_t rounds = sp.tiles / kSmCount, rest = sp.tiles % kSmCount;
  sp.full_tiles = (int)sp.tiles;
  sp.split = 1;
  double tail = rest ? 1.0 : 0.0;
  if (allow_split && rest > 0 && sp.tiles < (1 << 20)) {
    int64_t s = kSmCount / rest;
    if (s > kMaxSplit) s = kMaxSplit;
    while (s > 1 && kblocks / s < kMinSliceBlocks) --s;
    if (s >= 2) {
      sp.split = (int)s;
      sp.full_tiles = (int)(rounds * kSmCount);
      tail = 1.0 / s + 0.08;  // the exchange of partial tiles through L2
    }
  }
  const double w = bn == 256 ? penalty[0] : bn == 192 ? penalty[1] : penalty[2];
  sp.cost = ((double)rounds + tail) * bn * w;
  sp.scratch = sp.split > 1 ? 256 + (size_t)rest * 4 * sizeof(int) + 256 + (size_t)rest * sp.split * BM * bn * sizeof(float) : 0;
  return sp;
}

SplitPlan choose_plan(int64_t m, int64_t n, int64_t k, int kind, size_t scratch_bytes, bool unlimited) {
  const int64_t bk = kind == KIND_TF32 ? 32 : 64, kblocks = (k + bk - 1) / bk;
  SplitPlan best{};
  const int widths[3] = {256, 192, 128};
  for (int i = 0; i < 3; ++i) {
    SplitPlan sp = split_plan(widths[i], m, n, kblocks, true);
    if (!unlimited && sp.scratch > scratch_bytes) sp = split_plan(widths[i], m, n, kblocks, false);
    if (i == 0 || sp.cost < best.cost) best = sp;
  }
  return best;
}

template <int BN, int KIND>
int launch_tile(const void* a, const void* b, const void* bias, void* c, int out_dtype, int64_t m, int64_t n, int64_t k,
                int transpose_b, int act, int32_t* status, const SplitPlan& sp, void* scratch, cudaStream_t s) {
  constexpr int BK = KindCfg<KIND>::BK, NBOX = KROW_BYTES / KindCfg<KIND>::ESZ;
  EncodeTiledFn enc;
  if (int rc = get_encoder(&enc)) return rc;
  CUtensorMap map_a, map_b;
  if (int rc = make_map(enc, &map_a, a, KIND, m, k, BM, BK)) return rc;
  if (transpose_b) {
    if (int rc = make_map(enc, &map_b, b, KIND, n, k, BN, BK)) return rc;  // [N,K]: box BN rows x one K block
  } else {
    if (int rc = make_map(enc, &map_b, b, KIND, k, n, BK, NBOX)) return rc;  // [K,N]: box BK rows x 128 bytes of N
  }
  GemmParams p{(int)m, (int)n, (int)k, transpose_b ? 1 : 0, act, bias, c, status, sp.full_tiles, sp.split, nullptr, nullptr};
  int64_t units = sp.tiles;
  if (sp.split > 1) {
    const int64_t rest = sp.tiles - sp.full_tiles;
    char* base = static_cast<char*>(scratch);
    p.tickets = reinterpret_cast<int*>(base);
    p.partial = reinterpret_cast<float*>(base + ((256 + (size_t)rest * 4 * sizeof(int) + 255) & ~(size_t)255));
    units = sp.full_tiles + rest * sp.split;
    // whatever used this scratch before (another plan sharing the workspace) may have left anything in the tickets
    IB200_CUDA_OK(cudaMemsetAsync(p.tickets, 0, (size_t)rest * 4 * sizeof(int), s));
  }
  const int grid = (int)(units < kSmCount ? units : kSmCount);
  void (*kern)(const CUtensorMap, const CUtensorMap, const GemmParams) = nullptr;
  if (KIND == KIND_BF16) kern = out_dtype == IB200_BF16 ? gemm_tcgen05_kernel<__nv_bfloat16, BN, KIND> : gemm_tcgen05_kernel<float, BN, KIND>;
  else if (KIND == KIND_F16) kern = out_dtype == IB200_F16 ? gemm_tcgen05_kernel<__half, BN, KIND> : gemm_tcgen05_kernel<float, BN, KIND>;
  else kern = gemm_tcgen05_kernel<float, BN, KIND>;
  IB200_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, TileCfg<BN>::SMEM));
  kern<<<grid, GEMM_THREADS, TileCfg<BN>::SMEM, s>>>(map_a, map_b, p);
  return cudaPeekAtLastError() == cudaSuccess ? IB200_OK : cuda_fail(cudaGetLastError(), "gemm tcgen05 launch");
}

template <int KIND>
int launch_pair(const void* a, const void* b, const void* bias, void* c, int out_dtype, int64_t m, int64_t n, int64_t k, int transpose_b,
                int act, int32_t* status, cudaStream_t s, int flags) {
  constexpr int BN = 256, BK = KindCfg<KIND>::BK, NBOX = KROW_BYTES / KindCfg<KIND>::ESZ;
  EncodeTiledFn enc;
  if (int rc = get_encoder(&enc)) return rc;
  CUtensorMap map_a, map_b;
  if (int rc = make_map(enc, &map_a, a, KIND, m, k, BM, BK)) return rc;
  if (transpose_b) {
    if (int rc = make_map(enc, &map_b, b, KIND, n, k, BN / 2, BK)) return rc;  // [N,K]: box of one CTA's half of the columns x one K block
  } else {
    if (int rc = make_map(enc, &map_b, b, KIND, k, n, BK, NBOX)) return rc;
  }
  CUtensorMap map_b_narrow = map_b;  // [N,K] operands: the box of a half-width unit (a [K,N] operand is loaded in 128-byte boxes either way)
  if (transpose_b) {
    if (int rc = make_map(enc, &map_b_narrow, b, KIND, n, k, BN / 4, BK)) return rc;
  }
  const int64_t tiles = ((m + 2 * BM - 1) / (2 * BM)) * ((n + BN - 1) / BN);
  const int pairs = (int)(tiles < kSmCount / 2 ? tiles : kSmCount / 2);
  const int64_t tail = tiles % pairs;
  const int narrow_from = (int)((flags & IB200_GEMM_NARROW_TAIL) != 0 && tail > 0 && 2 * tail <= pairs ? tiles - tail : tiles);
  GemmParams p{(int)m, (int)n, (int)k, transpose_b ? 1 : 0, act, bias, c, status, 0, 1, nullptr, nullptr, narrow_from};
  void (*kern)(const CUtensorMap, const CUtensorMap, const CUtensorMap, const GemmParams) = nullptr;
  if (KIND == KIND_BF16) kern = out_dtype == IB200_BF16 ? gemm_tcgen05_pair_kernel<__nv_bfloat16, BN, KIND> : gemm_tcgen05_pair_kernel<float, BN, KIND>;
  else if (KIND == KIND_F16) kern = out_dtype == IB200_F16 ? gemm_tcgen05_pair_kernel<__half, BN, KIND> : gemm_tcgen05_pair_kernel<float, BN, KIND>;
  else kern = gemm_tcgen05_pair_kernel<float, BN, KIND>;
  IB200_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, PairCfg<BN>::SMEM));
  kern<<<2 * pairs, GEMM_THREADS, PairCfg<BN>::SMEM, s>>>(map_a, map_b, map_b_narrow, p);
  return cudaPeekAtLastError() == cudaSuccess ? IB200_OK : cuda_fail(cudaGetLastError(), "gemm tcgen05 (CTA pairs) launch");
}

template <int KIND>
int run_tcgen05(const void* a, const void* b, const void* bias, void* c, int out_dtype, int64_t m, int64_t n, int64_t k,
                int transpose_b, int act, int32_t* status, void* scratch, size_t scratch_bytes, cudaStream_t s, bool pair, int flags) {
  // tile width: fewest (rounds of 148 CTAs) x (time per tile); narrower tiles re-read A more often and
  // the main loop is bound by operand traffic into shared memory, so they only win when they
  // save whole rounds (small or ragged N)
  if (pair) return launch_pair<KIND>(a, b, bias, c, out_dtype, m, n, k, transpose_b, act, status, s, flags);
  if (!scratch || (reinterpret_cast<uintptr_t>(scratch) & 255u)) scratch_bytes = 0;
  const SplitPlan sp = choose_plan(m, n, k, KIND, scratch_bytes, false);
  switch (sp.bn) {
    case 192: return launch_tile<192, KIND>(a, b, bias, c, out_dtype, m, n, k, transpose_b, act, status, sp, scratch, s);
    case 128: return launch_tile<128, KIND>(a, b, bias, c, out_dtype, m, n, k, transpose_b, act, status, sp, scratch, s);
    default: return launch_tile<256, KIND>(a, b, bias, c, out_dtype, m, n, k, transpose_b, act, status, sp, scratch, s);
  }
}

// ============================== FMA path ==============================================
template <typename TIn, typename TOut>
__global__ void __launch_bounds__(256) gemm_fma_kernel(const TIn* __restrict__ A, const TIn* __restrict__ B,
                                                       const TOut* __restrict__ bias, TOut* __restrict__ C, int M, int N, int K,
                                                       int b_kmajor, int act) {
  constexpr int T = 64, KB = 16;
  __shared__ float sa[KB][T + 1], sb[KB][T + 1];
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  const int m0 = blockIdx.y * T, n0 = blockIdx.x * T;
  float acc[4][4] = {};
  for (int k0 = 0; k0 < K; k0 += KB) {
    for (int i = threadIdx.x; i < T * KB; i += 256) {
      {  // A tile: T rows x KB cols, read along K
        const int r = i / KB, kk = i % KB;
        const int gm = m0 + r, gk = k0 + kk;
        sa[kk][r] = (gm < M && gk < K) ? to_f32<TIn>(A[(size_t)gm * K + gk]) : 0.0f;
      }
      if (b_kmajor) {  // B stored [N,K]
        const int c = i / KB, kk = i % KB;
        const int gn = n0 + c, gk = k0 + kk;
        sb[kk][c] = (gn < N && gk < K) ? to_f32<TIn>(B[(size_t)gn * K + gk]) : 0.0f;
      } else {  // B stored [K,N], read along N
        const int kk = i / T, c = i % T;
        const int gn = n0 + c, gk = k0 + kk;
        sb[kk][c] = (gn < N && gk < K) ? to_f32<TIn>(B[(size_t)gk * N + gn]) : 0.0f;
      }
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < KB; ++kk) {
      float av[4], bv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) { av[i] = sa[kk][ty * 4 + i]; bv[i] = sb[kk][tx * 4 + i]; }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int gm = m0 + ty * 4 + i;
    if (gm >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int gn = n0 + tx * 4 + j;
      if (gn >= N) continue;
      float v = acc[i][j];
      if (bias) v += to_f32<TOut>(bias[gn]);
      if (act == IB200_ACT_RELU) v = max_nan(v, 0.0f);
      C[(size_t)gm * N + gn] = from_f32<TOut>(v);
    }
  }
}

template <typename TIn, typename TOut>
int run_fma(const void* a, const void* b, const void* bias, void* c, int64_t m, int64_t n, int64_t k, int transpose_b, int act,
            cudaStream_t s) {
  dim3 grid((unsigned)((n + 63) / 64), (unsigned)((m + 63) / 64));
  if (grid.y > 65535) return fail(IB200_ERR_UNSUPPORTED, "gemm (FMA path): M above 64*65535");
  gemm_fma_kernel<TIn, TOut><<<grid, 256, 0, s>>>(static_cast<const TIn*>(a), static_cast<const TIn*>(b),
                                                   static_cast<const TOut*>(bias), static_cast<TOut*>(c), (int)m, (int)n, (int)k,
                                                   transpose_b ? 1 : 0, act);
  return cudaPeekAtLastError() == cudaSuccess ? IB200_OK : cuda_fail(cudaGetLastError(), "gemm fma launch");
}

}  // namespace

bool gemm_uses_tensor_cores(int in_dtype, int out_dtype, int64_t n, int64_t k, int flags) {
  const bool in_ok = in_dtype == IB200_BF16 || in_dtype == IB200_F16 || (in_dtype == IB200_F32 && (flags & IB200_GEMM_ALLOW_TF32));
  const bool out_ok = out_dtype == IB200_F32 || (in_dtype != IB200_F32 && out_dtype == in_dtype);
  return in_ok && out_ok && k >= 8 && k % 8 == 0 && n % 8 == 0;
}

// CTA pairs (256 x 256 tiles) when the problem has rows for both CTAs of a pair and tiles for at least half of the
// 74 pairs: measured on 4096^3 bf16, 101.9 us against 108.7 us for the one-CTA kernel (8192^3: 821 against 968 us);
// smaller problems keep the one-CTA kernel, whose narrower tiles and K-split tail fill the SMs better
bool prefers_cta_pairs(int64_t m, int64_t n, int flags) {
  if (flags & IB200_GEMM_ONE_CTA) return false;
  if (flags & IB200_GEMM_CTA_PAIRS) return true;
  const int64_t tiles = ((m + 2 * BM - 1) / (2 * BM)) * ((n + 255) / 256);
  return m >= 2 * BM && tiles >= kSmCount / 4;
}

// a [K,N] f32 operand is transposed into the front of the scratch; the K-split area follows
size_t tf32_transpose_bytes(int64_t n, int64_t k) { return ((size_t)n * k * sizeof(float) + 255) & ~(size_t)255; }

size_t gemm_scratch_bytes(int in_dtype, int out_dtype, int64_t m, int64_t n, int64_t k, int flags, int transpose_b) {
  if (m <= 0 || n <= 0 || !gemm_uses_tensor_cores(in_dtype, out_dtype, n, k, flags)) return 0;
  const size_t split = prefers_cta_pairs(m, n, flags) ? 0 : choose_plan(m, n, k, in_dtype == IB200_F32 ? KIND_TF32 : KIND_BF16, 0, true).scratch;
  return split + (in_dtype == IB200_F32 && !transpose_b ? tf32_transpose_bytes(n, k) : 0);
}

int launch_gemm(const void* a, const void* b, const void* bias, void* c, int in_dtype, int out_dtype, int64_t m, int64_t n,
                int64_t k, int transpose_b, int act, int32_t* status, cudaStream_t s, int flags, void* scratch, size_t scratch_bytes) {
  if (m < 0 || n < 0 || k < 0) return fail(IB200_ERR_INVALID, "gemm: negative extent");
  if (m == 0 || n == 0) return IB200_OK;
  if (beyond_any_device(m, n) || beyond_any_device(m, k > 0 ? k : 1) || beyond_any_device(k > 0 ? k : 1, n))
    return fail(IB200_ERR_INVALID, "gemm: more than 2^40 elements in an operand");
  if (!a || !b || !c) {
    if (k > 0 || !c) return fail(IB200_ERR_INVALID, "gemm: null pointer");
  }
  if (m > INT32_MAX || n > INT32_MAX || k > INT32_MAX) return fail(IB200_ERR_UNSUPPORTED, "gemm: extent above 2^31-1");
  if (act != IB200_ACT_NONE && act != IB200_ACT_RELU) return fail(IB200_ERR_INVALID, "gemm: unknown activation");
  bool tc = gemm_uses_tensor_cores(in_dtype, out_dtype, n, k, flags) && aligned16(a) && aligned16(b) && aligned16(c) &&
            (!bias || aligned16(bias));
  if (!scratch || (reinterpret_cast<uintptr_t>(scratch) & 255u)) scratch_bytes = 0;
  if (tc && in_dtype == IB200_F32 && !transpose_b) {  // TF32 takes B as [N,K]: transpose it into the scratch, or stay on the FMA kernel
    const size_t need = tf32_transpose_bytes(n, k);
    if (scratch_bytes < need) {
      tc = false;
    } else {
      if (int rc = launch_transpose2d(b, scratch, 4, k, n, s)) return rc;
      b = scratch;
      transpose_b = 1;
      scratch = static_cast<char*>(scratch) + need;
      scratch_bytes -= need;
    }
  }
  if (tc) {
    if (!status) return fail(IB200_ERR_INVALID, "gemm: the tensor-core path needs a device status word");
    const bool pair = prefers_cta_pairs(m, n, flags);
    if (in_dtype == IB200_BF16) return run_tcgen05<KIND_BF16>(a, b, bias, c, out_dtype, m, n, k, transpose_b, act, status, scratch, scratch_bytes, s, pair, flags);
    if (in_dtype == IB200_F16) return run_tcgen05<KIND_F16>(a, b, bias, c, out_dtype, m, n, k, transpose_b, act, status, scratch, scratch_bytes, s, pair, flags);
    return run_tcgen05<KIND_TF32>(a, b, bias, c, out_dtype, m, n, k, transpose_b, act, status, scratch, scratch_bytes, s, pair, flags);
  }
  if (in_dtype == IB200_F32 && out_dtype == IB200_F32) return run_fma<float, float>(a, b, bias, c, m, n, k, transpose_b, act, s);
  if (in_dtype == IB200_BF16 && out_dtype == IB200_BF16) return run_fma<__nv_bfloat16, __nv_bfloat16>(a, b, bias, c, m, n, k, transpose_b, act, s);
  if (in_dtype == IB200_BF16 && out_dtype == IB200_F32) return run_fma<__nv_bfloat16, float>(a, b, bias, c, m, n, k, transpose_b, act, s);
  if (in_dtype == IB200_F32 && out_dtype == IB200_BF16) return run_fma<float, __nv_bfloat16>(a, b, bias, c, m, n, k, transpose_b, act, s);
  if (in_dtype == IB200_F16 && out_dtype == IB200_F16) return run_fma<__half, __half>(a, b, bias, c, m, n, k, transpose_b, act, s);
  if (in_dtype == IB200_F16 && out_dtype == IB200_F32) return run_fma<__half, float>(a, b, bias, c, m, n, k, transpose_b, act, s);
  return fail(IB200_ERR_UNSUPPORTED, "gemm: operand dtypes must be f32, f16 or bf16");
}

}  // namespace ib200
