// FP32 GEMM on the tensor cores, CTA-pair form of k_gemm_tf32x3.cu: the same 3xTF32
// split, TMA feed, TMEM accumulators and fused epilogue, but two CTAs of a cluster share
// one 256 x 256 tile through tcgen05.mma.cta_group::2.  Each CTA stages, splits and feeds
// only its 128 rows of A and its 128 columns of B (half the B tile of the single-CTA
// kernel), which is what relieves shared-memory bandwidth, the co-limiter measured there.
//
// Pair protocol (rank = %cluster_ctarank, rank 0 leads):
//   * both CTAs allocate tensor memory with cta_group::2; each holds the accumulator rows of
//     its own 128 A rows for all 256 columns, double-buffered (512 columns);
//   * TMA producer, converters and epilogue run in both CTAs on local barriers;
//   * converters of both CTAs arrive on the LEADER's full_cvt barrier (remote arrive through
//     mapa, release at cluster scope; count 2 x 128);
//   * only the leader's MMA thread issues; its commits are multicast to both CTAs' `empty`
//     (stage reusable) and `acc_full` (tile done) barriers;
//   * epilogue threads of both CTAs arrive on the leader's acc_empty barrier (2 x 128).
// Every wait is bounded; each CTA times out on its own and the pair meets at a cluster
// barrier before tensor memory is released.
#include <cuda.h>
#include <cudaTypedefs.h>

#include <cstdlib>

#include "k_epilogue.cuh"
#include "k_umma.cuh"
#include "ta_core.hpp"

namespace ta {

namespace {

using namespace umma;

constexpr int BM = 128;                    // rows per CTA (the pair covers 256)
constexpr int BNH = 128;                   // B columns per CTA (the pair covers 256)
constexpr int BN = 256;
constexpr int BK = 16;
constexpr int CVT_GROUPS = 2;
// warpgroups (4 warps each) as in the single-CTA kernel: 0-1 epilogue (left / right half of the
// tile's columns, running sums in registers), 2 = TMA warp + MMA warp + two idle warps, 3-4 converters
constexpr int EPI_WARPS = 8, TMA_WARP = 8, MMA_WARP = 9, CVT_WARP0 = 12;
constexpr int NUM_THREADS = (CVT_WARP0 + 4 * CVT_GROUPS) * 32;   // 640
constexpr uint32_t CHUNK_KB = 38;           // most K blocks (608 k) one tensor-memory accumulation absorbs
constexpr int LAUNCH_REGS = 96, EPI_REGS = 168, WORKER_REGS = 48;
static_assert(EPI_WARPS * 32 * EPI_REGS + (NUM_THREADS - EPI_WARPS * 32) * WORKER_REGS <= NUM_THREADS * LAUNCH_REGS,
              "setmaxnreg split exceeds the CTA's launch-time register allocation");
static_assert(NUM_THREADS * (LAUNCH_REGS + 8) > 65536, "LAUNCH_REGS must be what __launch_bounds__ yields");
constexpr int A_BYTES = BM * BK * 4;       // 8 KiB
constexpr int B_BYTES = BK * BNH * 4;      // 8 KiB
constexpr int HALF_BYTES = A_BYTES + B_BYTES;
constexpr int STAGE_BYTES = 2 * HALF_BYTES;   // hi (raw) + lo
constexpr int STAGES = 6;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 256 + 1024;
constexpr int TMEM_COLS = 512;
constexpr int ACC_STRIDE = 256;

__device__ __forceinline__ uint32_t split_lo(float x) {
  const float hi = __uint_as_float(__float_as_uint(x) & 0xffffe000u);
  return (__float_as_uint(x - hi) + 0x1000u) & 0xffffe000u;
}
__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// address of `local_bar` in the leader CTA's shared memory
__device__ __forceinline__ uint32_t leader_addr(uint32_t local_bar) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_bar), "r"(0u));
  return r;
}
__device__ __forceinline__ void mbar_arrive_remote(uint32_t cluster_bar) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait_cluster(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool mbar_wait_cluster(uint32_t bar, uint32_t parity, volatile uint32_t *abort,
                                                  uint32_t sleep_ns = 0) {
  if (mbar_try_wait_cluster(bar, parity)) return true;
  const uint64_t t0 = global_timer_ns();
  uint32_t spins = 0;
  while (!mbar_try_wait_cluster(bar, parity)) {
    if (sleep_ns) __nanosleep(sleep_ns);
    if ((++spins & 63u) == 0) {
      if (*abort) return false;
      if (global_timer_ns() - t0 > WAIT_LIMIT_NS) {
        *abort = 1;
        return false;
      }
    }
  }
  return true;
}
__device__ __forceinline__ void tmem_alloc2(uint32_t smem_dst, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(cols) : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc2(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
// completion of all earlier MMAs of this thread -> one arrival on `bar` in BOTH CTAs of the pair
__device__ __forceinline__ void tc_commit_pair(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(bar), "h"((uint16_t)3) : "memory");
}
__device__ __forceinline__ void mma_tf32_pair(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                              uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::tf32 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}

__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_tf32x3_pair_kernel(const GemmParams p, const __grid_constant__ CUtensorMap map_a,
                        const __grid_constant__ CUtensorMap map_b, uint32_t *__restrict__ status) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t *smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t bar_base = smem_base + STAGES * STAGE_BYTES;
  auto full_raw = [&](int s) { return bar_base + 8u * s; };
  auto full_cvt = [&](int s) { return bar_base + 8u * (STAGES + s); };       // used in the leader
  auto empty = [&](int s) { return bar_base + 8u * (2 * STAGES + s); };
  auto acc_full = [&](int b) { return bar_base + 8u * (3 * STAGES + b); };
  auto acc_empty = [&](int b) { return bar_base + 8u * (3 * STAGES + 2 + b); };   // used in the leader
  volatile uint32_t *tmem_slot =
      reinterpret_cast<volatile uint32_t *>(smem_gen + STAGES * STAGE_BYTES + 8 * (3 * STAGES + 4));
  volatile uint32_t *abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_rank();
  const uint32_t pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_raw(s), 1);
      mbar_init(full_cvt(s), 256);    // one converter group of each CTA
      mbar_init(empty(s), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(acc_full(b), 1);
      mbar_init(acc_empty(b), 2 * EPI_WARPS * 32);   // the epilogue threads of both CTAs
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == MMA_WARP) tmem_alloc2(smem_u32((const void *)tmem_slot), TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();   // both CTAs' barriers exist before anyone arrives remotely
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const uint32_t tiles_m = (p.m + 2 * BM - 1) / (2 * BM), tiles_n = (p.n + BN - 1) / BN;
  const uint32_t tiles_per_batch = tiles_m * tiles_n;
  const uint32_t num_tiles = tiles_per_batch * p.batch;
  const uint32_t k_blocks = (p.k + BK - 1) / BK;

  const int wgroup = warp >> 2;
  if (wgroup == 2) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(WORKER_REGS));
  if (warp == TMA_WARP) {
    // ------------------------------------------------------------ TMA producer (both CTAs)
    uint32_t stage = 0, phase = 0;
    bool ok = true;
    for (uint32_t tile = pair; ok && tile < num_tiles; tile += num_pairs) {
      const uint32_t batch = tile / tiles_per_batch, rem = tile % tiles_per_batch;
      const int m0 = (int)(rem / tiles_n) * 2 * BM + (int)rank * BM;
      const int n0 = (int)(rem % tiles_n) * BN + (int)rank * BNH;
      const int za = p.stride_a ? (int)batch : 0, zb = p.stride_b ? (int)batch : 0;
      for (uint32_t kb = 0; kb < k_blocks; ++kb) {
        ok = mbar_wait_cluster(empty(stage), phase ^ 1u, abort_flag);
        if (!ok) break;
        const uint32_t dst = smem_base + stage * STAGE_BYTES;
        if (elect_one()) {
          mbar_arrive_expect_tx(full_raw(stage), HALF_BYTES);
          tma_load_3d(dst, &map_a, full_raw(stage), (int)(kb * BK), m0, za);
          if (p.b_grouped) {
            tma_load_4d(dst + A_BYTES, &map_b, full_raw(stage), 0, (int)(kb * BK), n0 / 32, zb);
          } else {
#pragma unroll
            for (int nb = 0; nb < BNH / 32; ++nb)
              tma_load_3d(dst + A_BYTES + nb * (BK * 128), &map_b, full_raw(stage), n0 + nb * 32,
                          (int)(kb * BK), zb);
          }
        }
        __syncwarp();
        if (++stage == STAGES) { stage = 0; phase ^= 1u; }
      }
    }
  } else if (warp == MMA_WARP && rank == 0) {
    // ------------------------------------------------------------ MMA issuer (leader only)
    const uint32_t idesc = (1u << 4) | (2u << 7) | (2u << 10) | (1u << 16) |
                           ((uint32_t)(BN >> 3) << 17) | ((uint32_t)((2 * BM) >> 4) << 24);
    uint32_t stage = 0, phase = 0, acc_it = 0;
    bool ok = true;
    for (uint32_t tile = pair; ok && tile < num_tiles; tile += num_pairs) {
      for (uint32_t kb0 = 0; ok && kb0 < k_blocks; kb0 += p.chunk_kb, ++acc_it) {
        // one K chunk per tensor-memory buffer: the epilogue warps drain chunk c while chunk c+1 runs
        const uint32_t kb1 = min(k_blocks, kb0 + p.chunk_kb);
        const uint32_t buf = acc_it & 1u, acc_phase = (acc_it >> 1) & 1u;
        ok = mbar_wait_cluster(acc_empty(buf), acc_phase ^ 1u, abort_flag);
        if (!ok) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + buf * ACC_STRIDE;
        for (uint32_t kb = kb0; kb < kb1; ++kb) {
          ok = mbar_wait_cluster(full_cvt(stage), phase, abort_flag);
          if (!ok) break;
          tc_fence_after();
          const uint32_t a_hi = smem_base + stage * STAGE_BYTES;
          const uint32_t b_hi = a_hi + A_BYTES;
          const uint64_t da_hi0 = make_desc(a_hi, 16, 512, LAYOUT_SW64);
          const uint64_t da_lo0 = make_desc(a_hi + HALF_BYTES, 16, 512, LAYOUT_SW64);
          const uint64_t db_hi0 = make_desc(b_hi, BK * 128, 512, LAYOUT_SW128_BASE32B);
          const uint64_t db_lo0 = make_desc(b_hi + HALF_BYTES, BK * 128, 512, LAYOUT_SW128_BASE32B);
          if (elect_one()) {
#pragma unroll
            for (int j = 0; j < BK / 8; ++j) {
              const uint64_t da_hi = da_hi0 + (uint64_t)(j * 2), da_lo = da_lo0 + (uint64_t)(j * 2);
              const uint64_t db_hi = db_hi0 + (uint64_t)(j * 64), db_lo = db_lo0 + (uint64_t)(j * 64);
              mma_tf32_pair(d_tmem, da_lo, db_hi, idesc, ((kb - kb0) | (uint32_t)j) != 0u);
              mma_tf32_pair(d_tmem, da_hi, db_lo, idesc, 1u);
              mma_tf32_pair(d_tmem, da_hi, db_hi, idesc, 1u);
            }
            tc_commit_pair(empty(stage));
            if (kb + 1 == kb1) tc_commit_pair(acc_full(buf));
          }
          __syncwarp();
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
      }
    }
  }
  } else if (wgroup >= 3) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(WORKER_REGS));
    // ------------------------------------------------------------ hi/lo converters (both CTAs)
    const int t = (threadIdx.x - CVT_WARP0 * 32) & 127, group = (threadIdx.x - CVT_WARP0 * 32) >> 7;
    uint32_t stage = 0, phase = 0, it_all = 0;
    bool ok = true;
    for (uint32_t tile = pair; ok && tile < num_tiles; tile += num_pairs) {
      for (uint32_t kb = 0; kb < k_blocks; ++kb, ++it_all) {
        if ((int)(it_all % CVT_GROUPS) == group) {
          ok = mbar_wait(full_raw(stage), phase, abort_flag);
          if (!ok) break;
          float4 *hi = reinterpret_cast<float4 *>(smem_gen + stage * STAGE_BYTES);
          float4 *lo = reinterpret_cast<float4 *>(smem_gen + stage * STAGE_BYTES + HALF_BYTES);
#pragma unroll 4
          for (int i = t; i < HALF_BYTES / 16; i += 128) {
            const float4 v = hi[i];
            uint4 l;
            l.x = split_lo(v.x); l.y = split_lo(v.y); l.z = split_lo(v.z); l.w = split_lo(v.w);
            *reinterpret_cast<uint4 *>(lo + i) = l;
          }
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
          mbar_arrive_remote(leader_addr(full_cvt(stage)));
        }
        if (++stage == STAGES) { stage = 0; phase ^= 1u; }
      }
    }
  } else {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(EPI_REGS));
    // ------------------------------------------------------------ epilogue (warps 0-7, both CTAs)
    // Warp w drains TMEM lanes 32 (w % 4) .. +31 (this CTA's tile rows) and the column half w / 4;
    // the chunks of a tile are summed in registers, as in the single-CTA kernel.
    constexpr int HALF_N = BN / 2;
    const int lane_grp = warp & 3, col_half = warp >> 2;
    uint32_t acc_it = 0;
    bool ok = true;
    const bool alpha_is_one = p.alpha == 1.0f;
    for (uint32_t tile = pair; ok && tile < num_tiles; tile += num_pairs) {
      const uint32_t batch = tile / tiles_per_batch, rem = tile % tiles_per_batch;
      const uint32_t m0 = (rem / tiles_n) * 2 * BM + rank * BM, n0 = (rem % tiles_n) * BN + col_half * HALF_N;
      float sum[HALF_N];
#pragma unroll
      for (int i = 0; i < HALF_N; ++i) sum[i] = 0.0f;
      for (uint32_t kb0 = 0; ok && kb0 < k_blocks; kb0 += p.chunk_kb, ++acc_it) {
        const uint32_t buf = acc_it & 1u, acc_phase = (acc_it >> 1) & 1u;
        ok = mbar_wait_cluster(acc_full(buf), acc_phase, abort_flag, 256);
        if (!ok) break;
        tc_fence_after();
        const uint32_t taddr = tmem_base + buf * ACC_STRIDE + col_half * HALF_N + ((uint32_t)(lane_grp * 32) << 16);
#pragma unroll
        for (int c0 = 0; c0 < HALF_N; c0 += 16) {
          float v[16];
          tmem_ld16(taddr + c0, v);
#pragma unroll
          for (int i = 0; i < 16; ++i) sum[c0 + i] += v[i];
        }
        tc_fence_before();
        mbar_arrive_remote(leader_addr(acc_empty(buf)));
      }
      if (!ok) break;
      const uint32_t row = m0 + lane_grp * 32 + lane;
      const bool row_ok = row < p.m;
      const size_t row_off = (size_t)batch * p.stride_c + (size_t)row * p.n;
      float *__restrict__ crow = p.c + row_off;
      const float *__restrict__ drow = p.d ? p.d + row_off : nullptr;
      const float *__restrict__ bias = p.bias ? p.bias + (size_t)batch * p.bias_stride : nullptr;
      if (row_ok) {
        epi_dispatch_act(p.act, [&](auto act_tag) {
          constexpr uint32_t ACT = decltype(act_tag)::value;
#pragma unroll
          for (int q = 0; q < HALF_N; q += 4) {
            const uint32_t col = n0 + q;
            if (col < p.n) {  // N % 4 == 0: a float4 is either fully in or fully out
              float4 o = make_float4(sum[q], sum[q + 1], sum[q + 2], sum[q + 3]);
              if (!alpha_is_one) { o.x *= p.alpha; o.y *= p.alpha; o.z *= p.alpha; o.w *= p.alpha; }
              if (p.accumulate) {
                const float4 c_old = *reinterpret_cast<const float4 *>(crow + col);
                o.x += c_old.x; o.y += c_old.y; o.z += c_old.z; o.w += c_old.w;
              }
              float4 bv = make_float4(0.f, 0.f, 0.f, 0.f), dv = bv;
              if (bias) bv = __ldg(reinterpret_cast<const float4 *>(bias + col));
              if (drow) dv = *reinterpret_cast<const float4 *>(drow + col);
              o.x = epi_apply_t<ACT>(o.x, bias != nullptr, bv.x, p.binary, dv.x, p.beta);
              o.y = epi_apply_t<ACT>(o.y, bias != nullptr, bv.y, p.binary, dv.y, p.beta);
              o.z = epi_apply_t<ACT>(o.z, bias != nullptr, bv.z, p.binary, dv.z, p.beta);
              o.w = epi_apply_t<ACT>(o.w, bias != nullptr, bv.w, p.binary, dv.w, p.beta);
              *reinterpret_cast<float4 *>(crow + col) = o;
            }
          }
        });
      }
    }
  }

  // ------------------------------------------------------------ teardown
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    for (int i = 0; i < 64; ++i) __nanosleep(100000);   // let copies / MMAs in flight land
    if (threadIdx.x == 0) atomicOr(status, 1u);
    __syncthreads();
  }
  cluster_sync_all();   // neither CTA frees tensor memory or leaves while the other may still use the pair
  if (warp == MMA_WARP) {
    tc_fence_after();
    tmem_dealloc2(tmem_base, TMEM_COLS);
  }
}

}  // namespace

bool gemm_tf32x3_pair_supported(const GemmParams &p, int sm_count) {
  return gemm_tf32x3_eligible(p) && sm_count >= 2;
}

void launch_gemm_tf32x3_pair(const Context &ctx, const GemmParams &p_in, uint32_t *status, cudaStream_t stream) {
  GemmParams p = p_in;
  // equal chunks of at most CHUNK_KB blocks: the truncation error follows the longest chunk
  {
    const uint32_t cap = tunables().tf32x3_chunk_kb ? tunables().tf32x3_chunk_kb : CHUNK_KB;
    const uint32_t kb_all = (p.k + 15u) / 16u, chunks = (kb_all + cap - 1) / cap;
    p.chunk_kb = chunks ? (kb_all + chunks - 1) / chunks : cap;
  }
  if (!gemm_tf32x3_pair_supported(p, ctx.sm_count))
    fail("paired tf32x3 GEMM needs f32 operands with K and N multiples of 4");
  static bool attr_set[64] = {};
  if (!attr_set[ctx.device & 63]) {
    TA_CUDA(cudaFuncSetAttribute(gemm_tf32x3_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
    attr_set[ctx.device & 63] = true;
  }
  CUtensorMap map_a, map_b;
  const uint64_t ba = p.stride_a ? p.batch : 1, bb = p.stride_b ? p.batch : 1;
  encode_map3(ctx, &map_a, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, p.a, p.k, p.m, ba, (uint64_t)p.k * 4,
              p.stride_a ? (uint64_t)p.stride_a * 4 : (uint64_t)p.m * p.k * 4, BK, BM, CU_TENSOR_MAP_SWIZZLE_64B);
  const uint64_t b_batch_bytes = p.stride_b ? (uint64_t)p.stride_b * 4 : (uint64_t)p.k * p.n * 4;
  p.b_grouped = p.n % 32 == 0 ? 1u : 0u;
  if (p.b_grouped)   // one TMA per stage for this CTA's 128-column half of the B block
    encode_map_grouped(ctx, &map_b, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, p.b, 4, p.n, p.k, bb, b_batch_bytes, 32, BK,
                       BNH / 32, CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B);
  else
    encode_map3(ctx, &map_b, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, p.b, p.n, p.k, bb, (uint64_t)p.n * 4, b_batch_bytes, 32, BK,
                CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B);
  const uint64_t tiles = (uint64_t)((p.m + 2 * BM - 1) / (2 * BM)) * ((p.n + BN - 1) / BN) * p.batch;
  const uint32_t pairs = (uint32_t)std::min<uint64_t>(tiles, (uint64_t)ctx.sm_count / 2);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(pairs * 2, 1, 1);
  cfg.blockDim = dim3(NUM_THREADS, 1, 1);
  cfg.dynamicSmemBytes = SMEM_BYTES;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  TA_CUDA(cudaLaunchKernelEx(&cfg, gemm_tf32x3_pair_kernel, p, map_a, map_b, status));
  g_launches.fetch_add(1, std::memory_order_relaxed);
}

}  // namespace ta
