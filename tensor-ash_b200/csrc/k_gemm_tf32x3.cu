// FP32 GEMM on the 5th-generation tensor cores: TMA-fed, tcgen05.mma kind::tf32
// with a 3-pass split (3xTF32), f32 accumulators in tensor memory, fused
// epilogue on the TMEM -> register drain.  Persistent: one CTA per SM walks a
// static tile schedule.
//
// What it computes is the reference's default FP32 GEMM
// (shaders/matmul_bda_v4_kernel.glsl:225-452 with the epilogue of
// shaders/matmul_epilogue_common.glsl:14-82):
//     C[b,i,j] = epi(alpha * sum_k A[b,i,k] * B[b,k,j] (+ C[b,i,j]))
// A [B,M,K], B [K,N] or [B,K,N], C/D [B,M,N] row-major f32, bias [N] or [B,N].
//
// Split: x = hi + lo with hi = trunc_tf32(x) (what the tensor core sees when it
// reads the raw f32 word) and lo = rn_tf32(x - hi) (x - hi is exact in f32).
// Per K step the tensor core adds  a_lo*b_hi + a_hi*b_lo + a_hi*b_hi  into one
// f32 accumulator; the dropped a_lo*b_lo term is below 2^-20 relative.  The
// split is elementwise, so the converter warps leave the TMA tile untouched (it
// is the hi operand) and write lo into a twin buffer at identical offsets: the
// shared-memory swizzle never has to be decoded.
//
// Warp roles (640 threads, five warpgroups): warps 0-7 drain TMEM and run the epilogue
// (warp w owns TMEM lanes 32 (w % 4).. = tile rows and the column half w / 4), warp 8 issues
// TMA, warp 9 owns the TMEM allocation and issues the MMAs, warps 12-19 split tiles into
// hi/lo in two groups of four that take alternate K blocks (one block's load-split-store-
// fence chain overlaps the next block's).  setmaxnreg moves registers from the worker
// warpgroups (48 each) to the epilogue warpgroups (168 each).
//
// Accuracy: the tensor-memory accumulator truncates after every MMA, an error that grows
// linearly with the number of MMAs one accumulation absorbs (measured worst case over 32 operand
// pairs, relative to max |C|: 4.8e-6 at 32 K blocks, 6.9e-6 at 43, 7.4e-6 at 44, 9.7e-6 at 64,
// 1.6e-5 when a whole K = 2048 runs in one accumulator).  K is therefore cut into equal chunks of at
// most 38 K blocks (608 k): a chunk accumulates in one of the two tensor-memory buffers, the
// epilogue warps drain it into per-thread running sums (round-to-nearest f32 adds) while the next
// chunk runs in the other buffer; a tile's epilogue runs on the running sums.  The error then
// stays under 6.5e-6 at any K, against the 1e-5 criterion.  Draining tensor memory takes bandwidth
// from the MMAs writing it (32 x 2048^3: 205 TFLOP/s with two chunks per tile, 202 with three), so
// the chunks are as long as the margin allows; the experiment switch tf32x3_chunk_kb sets the cap.
// Every mbarrier wait is bounded (about two seconds); on a timeout the CTA
// raises a flag, all roles leave their loops, and the host reports an error.
//
// SPLITK = true turns the same pipeline into stage 1 of the two-stage split-K route
// (src/executor/reduction.rs:21-70; shaders/matmul_splitk2_kernel.glsl:121-216 is the SIMT form):
// a work unit is (batch, output tile, K sub-range), the sub-range's product is accumulated in one
// tensor-memory buffer (at most 64 K blocks = 1024 k, so the truncating accumulator stays inside
// the chunk bound above) and alpha * partial is plain-stored to the unit's scratch plane; a
// separate kernel adds the planes in a fixed order.  The caller's split s covers K blocks
// [s KB/S, (s+1) KB/S) as the reference's partition does; each split is cut further into
// `c` equal sub-ranges so that units fill the machine whatever the requested split count.
#include <cuda.h>
#include <cudaTypedefs.h>

#include <cstdlib>

#include "k_epilogue.cuh"
#include "k_umma.cuh"
#include "ta_core.hpp"

namespace ta {

namespace {

constexpr int BM = 128;
constexpr int BK = 16;                      // floats per stage along K (64-byte rows of A)
constexpr int CVT_GROUPS = 2;               // converter groups of 4 warps, alternating K blocks
// warpgroups (4 warps each): 0-1 epilogue (left / right half of the tile's columns), 2 = TMA
// warp + MMA warp + two idle warps, 3-4 converters
constexpr int EPI_WARPS = 8, TMA_WARP = 8, MMA_WARP = 9, CVT_WARP0 = 12;
constexpr int NUM_THREADS = (CVT_WARP0 + 4 * CVT_GROUPS) * 32;   // 640
constexpr uint32_t CHUNK_KB = 38;           // most K blocks (608 k) one tensor-memory accumulation absorbs
// setmaxnreg only redistributes the registers the CTA was launched with (threads x the
// per-thread count the compiler reports, 96 for 640 threads), and `inc` blocks until they are
// there: the split must fit that pool or the kernel never starts.
constexpr int LAUNCH_REGS = 96, EPI_REGS = 168, WORKER_REGS = 48;
static_assert(EPI_WARPS * 32 * EPI_REGS + (NUM_THREADS - EPI_WARPS * 32) * WORKER_REGS <= NUM_THREADS * LAUNCH_REGS,
              "setmaxnreg split exceeds the CTA's launch-time register allocation");
static_assert(NUM_THREADS * (LAUNCH_REGS + 8) > 65536, "LAUNCH_REGS must be what __launch_bounds__ yields");

template <int BN>
struct Cfg {
  static constexpr int A_BYTES = BM * BK * 4;             // 8 KiB
  static constexpr int B_BYTES = BK * BN * 4;             // 16 KiB at BN = 256
  static constexpr int HALF_BYTES = A_BYTES + B_BYTES;    // hi (raw) region, then lo region
  static constexpr int STAGE_BYTES = 2 * HALF_BYTES;
  static constexpr int STAGES = (BN == 256) ? 4 : (BN == 128 ? 6 : 8);
  static constexpr int BAR_BYTES = 256;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + BAR_BYTES + 1024;  // +1024: manual alignment
  static constexpr int TMEM_COLS = 512;                   // two accumulator buffers at BN = 256
  static constexpr int ACC_STRIDE = (BN == 256) ? 256 : (BN == 128 ? 128 : 64);
};

using namespace umma;

// The tensor core reads an f32 word as tf32 by ignoring the low 13 mantissa bits
// (truncation toward zero, measured on B200).  So the raw tile IS the hi operand,
// hi = trunc_tf32(x), and only lo = x - hi has to be produced: exact in f32, then
// rounded to nearest tf32 with integer ops (add half an ulp, mask) so the tensor
// core's own truncation of lo loses nothing.  Four full-rate ALU ops per element.
__device__ __forceinline__ uint32_t split_lo(float x) {
  const float hi = __uint_as_float(__float_as_uint(x) & 0xffffe000u);
  return (__float_as_uint(x - hi) + 0x1000u) & 0xffffe000u;
}

// ---------------------------------------------------------------- kernel
template <int BN, bool SPLITK>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_tf32x3_kernel(const GemmParams p, const __grid_constant__ CUtensorMap map_a,
                   const __grid_constant__ CUtensorMap map_b, uint32_t *__restrict__ status) {
  using C = Cfg<BN>;
  if constexpr (SPLITK) {
    // the reduce kernel behind this one in the stream may be scheduled now; it waits for this
    // grid to finish before it reads a plane
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  }
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t *smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t bar_base = smem_base + C::STAGES * C::STAGE_BYTES;
  // barrier map (8 bytes each)
  auto full_raw = [&](int s) { return bar_base + 8u * s; };
  auto full_cvt = [&](int s) { return bar_base + 8u * (C::STAGES + s); };
  auto empty = [&](int s) { return bar_base + 8u * (2 * C::STAGES + s); };
  auto acc_full = [&](int b) { return bar_base + 8u * (3 * C::STAGES + b); };
  auto acc_empty = [&](int b) { return bar_base + 8u * (3 * C::STAGES + 2 + b); };
  volatile uint32_t *tmem_slot =
      reinterpret_cast<volatile uint32_t *>(smem_gen + C::STAGES * C::STAGE_BYTES + 8 * (3 * C::STAGES + 4));
  volatile uint32_t *abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < C::STAGES; ++s) {
      mbar_init(full_raw(s), 1);
      mbar_init(full_cvt(s), 128);
      mbar_init(empty(s), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(acc_full(b), 1);
      mbar_init(acc_empty(b), EPI_WARPS * 32);
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == MMA_WARP) tmem_alloc(smem_u32((const void *)tmem_slot), C::TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const uint32_t tiles_m = (p.m + BM - 1) / BM, tiles_n = (p.n + BN - 1) / BN;
  const uint32_t tiles_per_batch = tiles_m * tiles_n;
  const uint32_t k_blocks_all = (p.k + BK - 1) / BK;
  // split-K stage 1: a unit is (batch, tile, K sub-range); the sub-range index runs fastest
  const uint32_t subs = SPLITK ? p.sk_subs : 1u;
  const uint32_t num_tiles = tiles_per_batch * p.batch * subs;
  // unit -> batch, tile within the batch, K blocks [kb_lo, kb_hi)
  auto decode = [&](uint32_t unit, uint32_t &batch, uint32_t &rem, uint32_t &sub, uint32_t &kb_lo, uint32_t &kb_hi) {
    if constexpr (SPLITK) {
      sub = unit % subs;
      const uint32_t t = unit / subs;
      batch = t / tiles_per_batch;
      rem = t % tiles_per_batch;
      // sub-ranges never straddle a caller-visible split: split = sub / c, piece = sub % c
      const uint32_t split = sub / p.sk_c, piece = sub % p.sk_c;
      kb_lo = split * p.sk_kb_per_split + piece * p.sk_kb_per_sub;
      kb_hi = min((split + 1u) * p.sk_kb_per_split, kb_lo + p.sk_kb_per_sub);
    } else {
      sub = 0;
      batch = unit / tiles_per_batch;
      rem = unit % tiles_per_batch;
      kb_lo = 0;
      kb_hi = k_blocks_all;
    }
  };

  // Register budget by warpgroup (setmaxnreg is a warpgroup-wide instruction, so the split is on
  // warp / 4 first): the epilogue warpgroups keep a whole tile's running sums in registers,
  // everyone else needs few.
  const int wgroup = warp >> 2;
  if (wgroup == 2) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(WORKER_REGS));
  if (warp == TMA_WARP) {
    // ------------------------------------------------------------ TMA producer
    uint32_t stage = 0, phase = 0;
    bool ok = true;
    for (uint32_t tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x) {
      uint32_t batch, rem, sub, kb_lo, kb_hi;
      decode(tile, batch, rem, sub, kb_lo, kb_hi);
      const int m0 = (int)(rem / tiles_n) * BM, n0 = (int)(rem % tiles_n) * BN;
      const int za = p.stride_a ? (int)batch : 0, zb = p.stride_b ? (int)batch : 0;
      for (uint32_t kb = kb_lo; kb < kb_hi; ++kb) {
        ok = mbar_wait(empty(stage), phase ^ 1u, abort_flag);
        if (!ok) break;
        const uint32_t dst = smem_base + stage * C::STAGE_BYTES;
        if (elect_one()) {
          mbar_arrive_expect_tx(full_raw(stage), C::HALF_BYTES);
          tma_load_3d(dst, &map_a, full_raw(stage), (int)(kb * BK), m0, za);
          if (p.b_grouped) {
            tma_load_4d(dst + C::A_BYTES, &map_b, full_raw(stage), 0, (int)(kb * BK), n0 / 32, zb);
          } else {
#pragma unroll
            for (int nb = 0; nb < BN / 32; ++nb)
              tma_load_3d(dst + C::A_BYTES + nb * (BK * 128), &map_b, full_raw(stage), n0 + nb * 32,
                          (int)(kb * BK), zb);
          }
        }
        __syncwarp();
        if (++stage == C::STAGES) { stage = 0; phase ^= 1u; }
      }
    }
  } else if (warp == MMA_WARP) {
    // ------------------------------------------------------------ MMA issuer
    const uint32_t idesc = (1u << 4) | (2u << 7) | (2u << 10) | (1u << 16) |
                           ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
    uint32_t stage = 0, phase = 0, acc_it = 0;
    bool ok = true;
    for (uint32_t tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x) {
      uint32_t batch, rem, sub, kb_lo, kb_hi;
      decode(tile, batch, rem, sub, kb_lo, kb_hi);
      for (uint32_t kb0 = kb_lo; ok && kb0 < kb_hi; kb0 += p.chunk_kb, ++acc_it) {
        // one K chunk per tensor-memory buffer: the epilogue warps drain chunk c while chunk c+1 runs
        const uint32_t kb1 = min(kb_hi, kb0 + p.chunk_kb);
        const uint32_t buf = acc_it & 1u, acc_phase = (acc_it >> 1) & 1u;
        ok = mbar_wait(acc_empty(buf), acc_phase ^ 1u, abort_flag);
        if (!ok) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + buf * C::ACC_STRIDE;
        for (uint32_t kb = kb0; kb < kb1; ++kb) {
          ok = mbar_wait(full_cvt(stage), phase, abort_flag);
          if (!ok) break;
          tc_fence_after();
          // descriptors are built warp-uniformly; a K step of 8 floats moves A by 32 bytes (+2 in
          // the 16-byte address field) and MN-major B by 8 rows of 128 bytes (+64)
          const uint32_t a_hi = smem_base + stage * C::STAGE_BYTES;
          const uint32_t b_hi = a_hi + C::A_BYTES;
          const uint64_t da_hi0 = make_desc(a_hi, 16, 512, LAYOUT_SW64);
          const uint64_t da_lo0 = make_desc(a_hi + C::HALF_BYTES, 16, 512, LAYOUT_SW64);
          const uint64_t db_hi0 = make_desc(b_hi, BK * 128, 512, LAYOUT_SW128_BASE32B);
          const uint64_t db_lo0 = make_desc(b_hi + C::HALF_BYTES, BK * 128, 512, LAYOUT_SW128_BASE32B);
          if (elect_one()) {
#pragma unroll
            for (int j = 0; j < BK / 8; ++j) {
              const uint64_t da_hi = da_hi0 + (uint64_t)(j * 2), da_lo = da_lo0 + (uint64_t)(j * 2);
              const uint64_t db_hi = db_hi0 + (uint64_t)(j * 64), db_lo = db_lo0 + (uint64_t)(j * 64);
              mma_tf32(d_tmem, da_lo, db_hi, idesc, ((kb - kb0) | (uint32_t)j) != 0u);
              mma_tf32(d_tmem, da_hi, db_lo, idesc, 1u);
              mma_tf32(d_tmem, da_hi, db_hi, idesc, 1u);
            }
            tc_commit(empty(stage));                       // stage reusable once these MMAs retire
            if (kb + 1 == kb1) tc_commit(acc_full(buf));
          }
          __syncwarp();
          if (++stage == C::STAGES) { stage = 0; phase ^= 1u; }
        }
      }
    }
  }
  } else if (wgroup >= 3) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(WORKER_REGS));
    // ------------------------------------------------------------ hi/lo converters
    const int t = (threadIdx.x - CVT_WARP0 * 32) & 127, group = (threadIdx.x - CVT_WARP0 * 32) >> 7;
    uint32_t stage = 0, phase = 0, it_all = 0;
    bool ok = true;
    for (uint32_t tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x) {
      uint32_t batch, rem, sub, kb_lo, kb_hi;
      decode(tile, batch, rem, sub, kb_lo, kb_hi);
      for (uint32_t kb = kb_lo; kb < kb_hi; ++kb, ++it_all) {
        if ((int)(it_all % CVT_GROUPS) == group) {
          ok = mbar_wait(full_raw(stage), phase, abort_flag);
          if (!ok) break;
          float4 *hi = reinterpret_cast<float4 *>(smem_gen + stage * C::STAGE_BYTES);
          float4 *lo = reinterpret_cast<float4 *>(smem_gen + stage * C::STAGE_BYTES + C::HALF_BYTES);
#pragma unroll 4
          for (int i = t; i < C::HALF_BYTES / 16; i += 128) {
            const float4 v = hi[i];
            uint4 l;
            l.x = split_lo(v.x); l.y = split_lo(v.y); l.z = split_lo(v.z); l.w = split_lo(v.w);
            *reinterpret_cast<uint4 *>(lo + i) = l;
          }
          // generic-proxy writes -> visible to the tensor core's async-proxy reads
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
          mbar_arrive(full_cvt(stage));
        }
        if (++stage == C::STAGES) { stage = 0; phase ^= 1u; }
      }
    }
  } else {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(EPI_REGS));
    // ------------------------------------------------------------ epilogue (warps 0-7)
    // Warp w drains TMEM lanes 32 (w % 4) .. +31 (tile rows) and the column half w / 4.  The
    // chunks of a tile are summed in registers (ordinary round-to-nearest f32 adds), so the
    // truncating tensor-memory accumulator never absorbs more than one chunk of MMAs.
    constexpr int HALF_N = BN / 2;
    const int lane_grp = warp & 3, col_half = warp >> 2;
    uint32_t acc_it = 0;
    bool ok = true;
    const bool alpha_is_one = p.alpha == 1.0f;
    for (uint32_t tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x) {
      uint32_t batch, rem, sub, kb_lo, kb_hi;
      decode(tile, batch, rem, sub, kb_lo, kb_hi);
      const uint32_t m0 = (rem / tiles_n) * BM, n0 = (rem % tiles_n) * BN + col_half * HALF_N;
      float sum[HALF_N];
#pragma unroll
      for (int i = 0; i < HALF_N; ++i) sum[i] = 0.0f;
      for (uint32_t kb0 = kb_lo; ok && kb0 < kb_hi; kb0 += p.chunk_kb, ++acc_it) {
        const uint32_t buf = acc_it & 1u, acc_phase = (acc_it >> 1) & 1u;
        ok = mbar_wait(acc_full(buf), acc_phase, abort_flag, 256);
        if (!ok) break;
        tc_fence_after();
        const uint32_t taddr = tmem_base + buf * C::ACC_STRIDE + col_half * HALF_N + ((uint32_t)(lane_grp * 32) << 16);
#pragma unroll
        for (int c0 = 0; c0 < HALF_N; c0 += 16) {
          float v[16];
          tmem_ld16(taddr + c0, v);
#pragma unroll
          for (int i = 0; i < 16; ++i) sum[c0 + i] += v[i];
        }
        tc_fence_before();
        mbar_arrive(acc_empty(buf));
      }
      if (!ok) break;
      const uint32_t row = m0 + lane_grp * 32 + lane;
      const bool row_ok = row < p.m;
      if constexpr (SPLITK) {
        // alpha * partial to this unit's plane (plane = batch * subs + sub), nothing else
        float *__restrict__ prow = p.sk_planes + ((size_t)batch * subs + sub) * ((size_t)p.m * p.n) + (size_t)row * p.n;
        if (row_ok) {
#pragma unroll
          for (int q = 0; q < HALF_N; q += 4) {
            const uint32_t col = n0 + q;
            if (col < p.n) {
              float4 o = make_float4(sum[q], sum[q + 1], sum[q + 2], sum[q + 3]);
              if (!alpha_is_one) { o.x *= p.alpha; o.y *= p.alpha; o.z *= p.alpha; o.w *= p.alpha; }
              *reinterpret_cast<float4 *>(prow + col) = o;
            }
          }
        }
        continue;
      }
      const size_t row_off = (size_t)batch * p.stride_c + (size_t)row * p.n;
      float *__restrict__ crow = p.c + row_off;
      const float *__restrict__ drow = p.d ? p.d + row_off : nullptr;
      const float *__restrict__ bias = p.bias ? p.bias + (size_t)batch * p.bias_stride : nullptr;
      if (row_ok) {
        // one dispatch on the activation per tile; the store loop is compiled per activation
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
    // Give copies and MMAs still in flight a bounded time to land before the
    // shared and tensor memory they target is released.
    for (int i = 0; i < 64; ++i) __nanosleep(100000);
    if (threadIdx.x == 0) atomicOr(status, 1u);
    __syncthreads();
  }
  if (warp == MMA_WARP) {
    tc_fence_after();
    tmem_dealloc(tmem_base, C::TMEM_COLS);
  }
}

// ---------------------------------------------------------------- host side
void encode_map(const Context &ctx, CUtensorMap *map, const void *base, uint64_t d0, uint64_t d1,
                uint64_t d2, uint64_t stride1_bytes, uint64_t stride2_bytes, uint32_t box0,
                uint32_t box1, CUtensorMapSwizzle swz) {
  auto encode = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(ctx.encode_tiled);
  if (!encode) fail("cuTensorMapEncodeTiled is unavailable in this CUDA driver");
  const cuuint64_t dims[3] = {d0, d1, d2};
  const cuuint64_t strides[2] = {stride1_bytes, stride2_bytes};
  const cuuint32_t box[3] = {box0, box1, 1};
  const cuuint32_t estr[3] = {1, 1, 1};
  const CUresult rc = encode(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<void *>(base), dims,
                             strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swz,
                             CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (rc != CUDA_SUCCESS) fail("cuTensorMapEncodeTiled failed with CUresult %d", (int)rc);
}

template <int BN, bool SPLITK>
void launch_t(const Context &ctx, const GemmParams &p_in, uint32_t *status, cudaStream_t stream) {
  using C = Cfg<BN>;
  GemmParams p = p_in;
  // equal chunks of at most CHUNK_KB blocks: the truncation error follows the longest chunk
  {
    const uint32_t cap = tunables().tf32x3_chunk_kb ? tunables().tf32x3_chunk_kb : CHUNK_KB;
    const uint32_t kb_all = (p.k + 15u) / 16u, chunks = (kb_all + cap - 1) / cap;
    p.chunk_kb = chunks ? (kb_all + chunks - 1) / chunks : cap;
    if (SPLITK) p.chunk_kb = std::max(cap, p.sk_kb_per_sub);   // a unit's sub-range is one accumulation (the plan caps it)
  }
  static bool attr_set[64] = {};
  if (!attr_set[ctx.device & 63]) {
    TA_CUDA(cudaFuncSetAttribute(gemm_tf32x3_kernel<BN, SPLITK>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 C::SMEM_BYTES));
    attr_set[ctx.device & 63] = true;
  }
  CUtensorMap map_a, map_b;
  const uint64_t ba = p.stride_a ? p.batch : 1, bb = p.stride_b ? p.batch : 1;
  // A [ba, M, K]: dims innermost first {K, M, ba}; 64-byte rows in shared memory.
  encode_map(ctx, &map_a, p.a, p.k, p.m, ba, (uint64_t)p.k * 4,
             p.stride_a ? (uint64_t)p.stride_a * 4 : (uint64_t)p.m * p.k * 4, BK, BM,
             CU_TENSOR_MAP_SWIZZLE_64B);
  // B [bb, K, N]: dims {N, K, bb}; boxes of 32 columns (128 bytes) x BK rows.
  const uint64_t b_batch_bytes = p.stride_b ? (uint64_t)p.stride_b * 4 : (uint64_t)p.k * p.n * 4;
  p.b_grouped = p.n % 32 == 0 ? 1u : 0u;
  if (p.b_grouped)   // one TMA per stage for the whole BN-wide B block
    umma::encode_map_grouped(ctx, &map_b, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, p.b, 4, p.n, p.k, bb, b_batch_bytes, 32, BK,
                             BN / 32, CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B);
  else
    encode_map(ctx, &map_b, p.b, p.n, p.k, bb, (uint64_t)p.n * 4, b_batch_bytes, 32, BK,
               CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B);
  const uint64_t tiles = (uint64_t)((p.m + BM - 1) / BM) * ((p.n + BN - 1) / BN) * p.batch * (SPLITK ? p.sk_subs : 1u);
  const uint32_t grid = (uint32_t)std::min<uint64_t>(tiles, (uint64_t)ctx.sm_count);
  gemm_tf32x3_kernel<BN, SPLITK><<<grid, NUM_THREADS, C::SMEM_BYTES, stream>>>(p, map_a, map_b, status);
  TA_CUDA(cudaGetLastError());
  g_launches.fetch_add(1, std::memory_order_relaxed);
}

}  // namespace

// TMA needs 16-byte global strides and bases: K % 4 == 0, N % 4 == 0 (that
// also makes every batch stride a multiple of 16 bytes), f32 operands.
bool gemm_tf32x3_eligible(const GemmParams &p) {
  if (p.b_f16) return false;
  if (p.k % 4 || p.n % 4) return false;
  if ((reinterpret_cast<uintptr_t>(p.a) | reinterpret_cast<uintptr_t>(p.b) |
       reinterpret_cast<uintptr_t>(p.c)) & 15)
    return false;
  if (p.d && (reinterpret_cast<uintptr_t>(p.d) & 15)) return false;
  if (p.bias && (reinterpret_cast<uintptr_t>(p.bias) & 15)) return false;
  if ((p.stride_a % 4) || (p.stride_b % 4) || (p.stride_c % 4) || (p.bias_stride % 4)) return false;
  return true;
}

void launch_gemm_tf32x3(const Context &ctx, const GemmParams &p, uint32_t tile_n, uint32_t *status,
                        cudaStream_t stream) {
  if (!gemm_tf32x3_eligible(p)) fail("tf32x3 GEMM needs f32 operands with K and N multiples of 4");
  if (tile_n >= 256) launch_t<256, false>(ctx, p, status, stream);
  else launch_t<128, false>(ctx, p, status, stream);
}

// ---------------------------------------------------------------- K split of a lone few-tile GEMM
// A GEMM whose output tiles cover a fraction of the SMs (1024^3: 32 or 64 tiles on 148) leaves the
// rest idle for the whole K loop.  Such an op runs as the split-K stage 1 above over `c` equal K
// ranges per tile (planes of alpha * partial in the slot scratch) followed by one kernel that adds a
// tile's planes in plane order and applies the op's epilogue: same formulas, the sum's rounding
// order differs from the one-launch kernel's (shorter accumulations: the error is smaller).
namespace {
SplitK2TensorPlan ksplit_plan_for_width(uint32_t bn, uint32_t batch, uint32_t m, uint32_t n, uint32_t kb_all, int sm_count) {
  SplitK2TensorPlan plan;
  const uint64_t tiles = (uint64_t)((m + BM - 1) / BM) * ((n + bn - 1) / bn) * batch;
  if (tiles * 2 > (uint64_t)sm_count) return plan;                         // more than half a wave already
  uint64_t c = std::min<uint64_t>((uint64_t)sm_count / tiles, kb_all / 16); // a range keeps at least 256 k
  if (c < 2) return plan;
  c = std::max<uint64_t>(c, (kb_all + CHUNK_KB - 1) / CHUNK_KB);           // one accumulation holds at most CHUNK_KB blocks
  const uint32_t kb_per_sub = (uint32_t)((kb_all + c - 1) / c);
  c = (kb_all + kb_per_sub - 1) / kb_per_sub;
  plan.eligible = true;
  plan.tile_n = bn;
  plan.c = (uint32_t)c;
  plan.kb_per_split = kb_all;
  plan.kb_per_sub = kb_per_sub;
  plan.planes = (uint32_t)c;
  return plan;
}
}  // namespace

// Tile width: the one whose units (tiles x ranges) fill more of one wave; when the accumulation cap
// forces more ranges than a wave holds, the wider tile (fewer units).  Measured on 1024 x 512 x 1024
// (27.7 us at 256 wide, 21.6 at 128), 512 x 512 x 4096 (30.4 / 28.1) and 1024 x 1024 x 4096 (69.5 / 82.0).
SplitK2TensorPlan gemm_tf32x3_ksplit_plan(uint32_t batch, uint32_t m, uint32_t n, uint32_t k, int sm_count) {
  const int mode = tunables().tf32x3_ksplit;
  if (mode == 0 || k % BK != 0 || n % 4 != 0) return SplitK2TensorPlan{};
  if ((uint64_t)m * n * k < (1ull << 29)) return SplitK2TensorPlan{};      // small ops: the second launch costs more than it saves
  const uint32_t kb_all = k / BK;
  const SplitK2TensorPlan narrow = ksplit_plan_for_width(128, batch, m, n, kb_all, sm_count);
  if (mode == 128 || n % 256 != 0) return narrow;
  const SplitK2TensorPlan wide = ksplit_plan_for_width(256, batch, m, n, kb_all, sm_count);
  if (mode == 256 || !narrow.eligible) return wide;
  if (!wide.eligible) return narrow;
  const uint64_t sm = (uint64_t)sm_count;
  const uint64_t un = (uint64_t)((m + BM - 1) / BM) * ((n + 127) / 128) * batch * narrow.c;
  const uint64_t uw = (uint64_t)((m + BM - 1) / BM) * ((n + 255) / 256) * batch * wide.c;
  if (un <= sm && uw <= sm) return un > uw ? narrow : wide;
  return uw <= un ? wide : narrow;
}

size_t gemm_tf32x3_ksplit_scratch_bytes(uint32_t batch, uint32_t m, uint32_t n, uint32_t k, int sm_count) {
  const SplitK2TensorPlan plan = gemm_tf32x3_ksplit_plan(batch, m, n, k, sm_count);
  return plan.eligible ? (size_t)batch * plan.planes * m * n * 4 : 0;
}

namespace {
// One thread per four consecutive outputs of a row: planes in plane order from 0.0f, then
// (+ C_old) -> + bias -> activation -> binary stage, as the tile epilogues do.
template <uint32_t ACT>
__global__ void __launch_bounds__(256)
ksplit_reduce_epilogue_kernel(const float *__restrict__ planes, const GemmParams p, uint32_t nplanes) {
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const uint64_t mn = (uint64_t)p.m * p.n, total = mn * p.batch;
  const uint64_t base = ((uint64_t)blockIdx.x * blockDim.x + threadIdx.x) * 4;
  if (base >= total) return;
  const uint64_t batch = base / mn, e = base % mn;
  const uint32_t row = (uint32_t)(e / p.n), col = (uint32_t)(e % p.n);
  const float *src = planes + batch * nplanes * mn + e;
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  uint32_t s = 0;
  for (; s + 4 <= nplanes; s += 4) {
    float4 v[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) v[u] = __ldcg(reinterpret_cast<const float4 *>(src + (uint64_t)(s + u) * mn));
#pragma unroll
    for (int u = 0; u < 4; ++u) { acc.x += v[u].x; acc.y += v[u].y; acc.z += v[u].z; acc.w += v[u].w; }
  }
  for (; s < nplanes; ++s) {
    const float4 v = __ldcg(reinterpret_cast<const float4 *>(src + (uint64_t)s * mn));
    acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
  }
  const size_t off = (size_t)batch * p.stride_c + (size_t)row * p.n + col;
  if (p.accumulate) {
    const float4 c_old = *reinterpret_cast<const float4 *>(p.c + off);
    acc.x += c_old.x; acc.y += c_old.y; acc.z += c_old.z; acc.w += c_old.w;
  }
  float4 bv = make_float4(0.f, 0.f, 0.f, 0.f), dv = bv;
  if (p.bias) bv = __ldg(reinterpret_cast<const float4 *>(p.bias + (size_t)batch * p.bias_stride + col));
  if (p.d) dv = *reinterpret_cast<const float4 *>(p.d + off);
  const bool hb = p.bias != nullptr;
  acc.x = epi_apply_t<ACT>(acc.x, hb, bv.x, p.binary, dv.x, p.beta);
  acc.y = epi_apply_t<ACT>(acc.y, hb, bv.y, p.binary, dv.y, p.beta);
  acc.z = epi_apply_t<ACT>(acc.z, hb, bv.z, p.binary, dv.z, p.beta);
  acc.w = epi_apply_t<ACT>(acc.w, hb, bv.w, p.binary, dv.w, p.beta);
  *reinterpret_cast<float4 *>(p.c + off) = acc;
}

template <uint32_t ACT>
void launch_ksplit_reduce_t(const float *planes, const GemmParams &p, uint32_t nplanes, cudaStream_t stream) {
  const uint64_t threads = (uint64_t)p.batch * p.m * p.n / 4;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)((threads + 255) / 256), 1, 1);
  cfg.blockDim = dim3(256, 1, 1);
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;   // stage 1 releases its dependents at entry; this grid waits for it before the first plane read
  TA_CUDA(cudaLaunchKernelEx(&cfg, ksplit_reduce_epilogue_kernel<ACT>, planes, p, nplanes));
  g_launches.fetch_add(1, std::memory_order_relaxed);
}
}  // namespace

void launch_gemm_tf32x3_ksplit(const Context &ctx, const GemmParams &p_in, const SplitK2TensorPlan &plan, float *scratch,
                               uint32_t *status, cudaStream_t stream) {
  if (!plan.eligible || !gemm_tf32x3_eligible(p_in)) fail("internal: K-split 3xTF32 GEMM launched on an ineligible problem");
  GemmParams p = p_in;
  p.sk_subs = plan.planes;
  p.sk_c = plan.c;
  p.sk_kb_per_split = plan.kb_per_split;
  p.sk_kb_per_sub = plan.kb_per_sub;
  p.sk_planes = scratch;
  p.bias = nullptr; p.d = nullptr; p.accumulate = 0; p.act = 0; p.binary = 0;
  if (plan.tile_n >= 256) launch_t<256, true>(ctx, p, status, stream);
  else launch_t<128, true>(ctx, p, status, stream);
  switch (p_in.act) {
    case 1: launch_ksplit_reduce_t<1>(scratch, p_in, plan.planes, stream); break;
    case 2: launch_ksplit_reduce_t<2>(scratch, p_in, plan.planes, stream); break;
    case 3: launch_ksplit_reduce_t<3>(scratch, p_in, plan.planes, stream); break;
    default: launch_ksplit_reduce_t<0>(scratch, p_in, plan.planes, stream); break;
  }
}

// ---------------------------------------------------------------- split-K2 stage 1 on the tensor cores
// Eligible when the reference's partition (src/executor/splitk2.rs, shaders/matmul_splitk2_kernel.glsl:138-142:
// K / S per split, the first K % S splits one longer) lands on K-block boundaries: K a multiple
// of 16 * S.  Each split is then cut into c equal pieces of at most CHUNK_KB K blocks so that
// tiles * S * c work units fill the SMs whatever S the caller asked for; piece j of split s is
// plane s * c + j, and the reduce adds planes in that order.
SplitK2TensorPlan splitk2_tensor_plan(const GemmParams &p, uint32_t splits, int sm_count) {
  SplitK2TensorPlan plan;
  if (!tunables().splitk2_tensor || splits < 2 || p.b_f16 || !gemm_tf32x3_eligible(p)) return plan;
  if (p.k % (BK * splits) != 0 || p.m < 16 || p.n < 16) return plan;
  const uint32_t kb_per_split = p.k / BK / splits;
  const uint32_t bn = p.n <= 64 ? 64u : (p.n <= 128 || p.n % 256 != 0) ? 128u : 256u;
  const uint64_t tiles = (uint64_t)((p.m + BM - 1) / BM) * ((p.n + bn - 1) / bn) * p.batch;
  uint64_t c = std::max<uint64_t>(1, (uint64_t)sm_count / (tiles * splits));
  c = std::min<uint64_t>(c, kb_per_split);
  c = std::max<uint64_t>(c, (kb_per_split + CHUNK_KB - 1) / CHUNK_KB);   // one accumulation holds at most CHUNK_KB blocks
  const uint32_t kb_per_sub = (uint32_t)((kb_per_split + c - 1) / c);
  c = (kb_per_split + kb_per_sub - 1) / kb_per_sub;                      // no empty piece
  if ((uint64_t)splits * c > 65535) return plan;
  plan.eligible = true;
  plan.tile_n = bn;
  plan.c = (uint32_t)c;
  plan.kb_per_split = kb_per_split;
  plan.kb_per_sub = kb_per_sub;
  plan.planes = splits * (uint32_t)c;
  return plan;
}

void launch_splitk2_tensor(const Context &ctx, const GemmParams &p_in, const SplitK2TensorPlan &plan, float *scratch,
                           uint32_t *status, cudaStream_t stream) {
  if (!plan.eligible) fail("internal: tensor-core split-K stage 1 launched on an ineligible problem");
  GemmParams p = p_in;
  p.sk_subs = plan.planes;
  p.sk_c = plan.c;
  p.sk_kb_per_split = plan.kb_per_split;
  p.sk_kb_per_sub = plan.kb_per_sub;
  p.sk_planes = scratch;
  p.bias = nullptr; p.d = nullptr; p.accumulate = 0; p.act = 0; p.binary = 0;
  if (plan.tile_n >= 256) launch_t<256, true>(ctx, p, status, stream);
  else if (plan.tile_n >= 128) launch_t<128, true>(ctx, p, status, stream);
  else launch_t<64, true>(ctx, p, status, stream);
  launch_splitk2_reduce_wide(scratch, p.c, (uint64_t)p.batch * p.m * p.n, (uint64_t)p.m * p.n, plan.planes, stream);
}

}  // namespace ta
