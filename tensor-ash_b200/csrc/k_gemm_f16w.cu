// f16-weight GEMM on the tensor cores: C = epi(alpha * f16(A) @ B (+ C)) with
// A [B,M,K] f32, B [K,N] or [B,K,N] f16 (row-major, as uploaded), C/D f32.
// tcgen05.mma kind::f16 with f32 accumulation in tensor memory; the fused
// epilogue runs on the TMEM -> register drain.
//
// This is the tensor-core form of the reference's f16-weight tile kernels
// (shaders/matmul_bda_v4_kernel.glsl with B_IS_F16: f16 weights widened, f32
// accumulate; epilogue shaders/matmul_epilogue_common.glsl:14-82).  The one
// numeric difference: A is rounded to f16 (nearest-even) on its way into shared
// memory, because the tensor core multiplies f16 x f16.  Products are exact in
// f32 and accumulation is f32, so the error against the f64 oracle stays inside
// the f16-weight tolerance (2e-3 relative) -- a product's relative error grows
// from 2^-24 to at most 2^-11 and averages down over K.  |A| above 65504 would
// overflow f16; such inputs belong on the FFMA tiles (explicit kernel selection).
//
// Pipeline per K block of 32: TMA brings the raw f32 A tile (128 x 32, plain
// rows) and the f16 B tile (32 x BN, 128-byte swizzle, N-contiguous) into one
// stage; four converter warps turn the A tile into f16 in the 64-byte-swizzled
// K-major layout the tensor core reads; one thread issues two K=16 MMAs.
// Warps 0-3 drain TMEM (double-buffered accumulators), warp 4 is the TMA
// producer, warp 5 owns TMEM and issues MMAs, warps 6-13 convert (two groups of
// four warps taking alternate K blocks, so one block's load-convert-store-fence
// chain overlaps the next).  All waits are
// bounded; a timeout raises the abort flag and the host reports an error.
#include <cuda_fp16.h>

#include <cstdlib>

#include "k_epilogue.cuh"
#include "k_umma.cuh"
#include "ta_core.hpp"

namespace ta {

namespace {

using namespace umma;

constexpr int BM = 128;
constexpr int BK = 32;                     // K elements per stage
constexpr int CVT_GROUPS = 2;               // converter groups of 4 warps, alternating K blocks
constexpr int NUM_THREADS = 192 + CVT_GROUPS * 128;

template <int BN>
struct Cfg {
  static constexpr int RAW_BYTES = BM * BK * 4;           // 16 KiB f32 A tile
  static constexpr int A16_BYTES = BM * BK * 2;           // 8 KiB f16 A tile
  static constexpr int B_BYTES = BK * BN * 2;             // 16 KiB at BN = 256
  static constexpr int STAGE_BYTES = RAW_BYTES + A16_BYTES + B_BYTES;
  static constexpr int STAGES = (BN == 256) ? 5 : (BN == 128 ? 6 : 7);
  static constexpr int BAR_BYTES = 256;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + BAR_BYTES + 1024;
  static constexpr int TMEM_COLS = 2 * BN;                // 128, 256 or 512: powers of two
};

__device__ __forceinline__ uint32_t pack_half2(float a, float b) {
  const __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<const uint32_t *>(&h);
}

template <int BN>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_f16w_kernel(const GemmParams p, const __grid_constant__ CUtensorMap map_a,
                 const __grid_constant__ CUtensorMap map_b, uint32_t *__restrict__ status) {
  using C = Cfg<BN>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t *smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t bar_base = smem_base + C::STAGES * C::STAGE_BYTES;
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
      mbar_init(acc_empty(b), 128);
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 5) tmem_alloc(smem_u32((const void *)tmem_slot), C::TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const uint32_t tiles_m = (p.m + BM - 1) / BM, tiles_n = (p.n + BN - 1) / BN;
  const uint32_t tiles_per_batch = tiles_m * tiles_n;
  const uint32_t num_tiles = tiles_per_batch * p.batch;
  const uint32_t k_blocks = (p.k + BK - 1) / BK;

  if (warp == 4) {
    // ------------------------------------------------------------ TMA producer
    uint32_t stage = 0, phase = 0;
    bool ok = true;
    for (uint32_t tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x) {
      const uint32_t batch = tile / tiles_per_batch, rem = tile % tiles_per_batch;
      // M fastest: consecutive CTAs share one B column block (weights stream once through L2)
      const int m0 = (int)(rem % tiles_m) * BM, n0 = (int)(rem / tiles_m) * BN;
      const int za = p.stride_a ? (int)batch : 0, zb = p.stride_b ? (int)batch : 0;
      for (uint32_t kb = 0; kb < k_blocks; ++kb) {
        ok = mbar_wait(empty(stage), phase ^ 1u, abort_flag);
        if (!ok) break;
        if (lane == 0) {
          const uint32_t dst = smem_base + stage * C::STAGE_BYTES;
          mbar_arrive_expect_tx(full_raw(stage), C::RAW_BYTES + C::B_BYTES);
          tma_load_3d(dst, &map_a, full_raw(stage), (int)(kb * BK), m0, za);
#pragma unroll
          for (int nb = 0; nb < BN / 64; ++nb)
            tma_load_3d(dst + C::RAW_BYTES + C::A16_BYTES + nb * (BK * 128), &map_b, full_raw(stage),
                        n0 + nb * 64, (int)(kb * BK), zb);
        }
        __syncwarp();
        if (++stage == C::STAGES) { stage = 0; phase ^= 1u; }
      }
    }
  } else if (warp == 5) {
    // ------------------------------------------------------------ MMA issuer
    // c f32 | a,b f16 | a K-major, b N-major | N >> 3 | M >> 4
    const uint32_t idesc = (1u << 4) | (1u << 16) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
    uint32_t stage = 0, phase = 0, acc_it = 0;
    bool ok = true;
    for (uint32_t tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x, ++acc_it) {
      const uint32_t buf = acc_it & 1u, acc_phase = (acc_it >> 1) & 1u;
      ok = mbar_wait(acc_empty(buf), acc_phase ^ 1u, abort_flag);
      if (!ok) break;
      tc_fence_after();
      const uint32_t d_tmem = tmem_base + buf * BN;
      for (uint32_t kb = 0; kb < k_blocks; ++kb) {
        ok = mbar_wait(full_cvt(stage), phase, abort_flag);
        if (!ok) break;
        tc_fence_after();
        if (lane == 0) {
          const uint32_t a16 = smem_base + stage * C::STAGE_BYTES + C::RAW_BYTES;
          const uint32_t b16 = a16 + C::A16_BYTES;
#pragma unroll
          for (int j = 0; j < BK / 16; ++j) {
            // A: 64-byte rows, 8-row groups 512 B apart; B: 128-byte rows per k, 8-k groups 1 KiB
            // apart, 64-column blocks BK*128 B apart
            const uint64_t da = make_desc(a16 + j * 32, 16, 512, LAYOUT_SW64);
            const uint64_t db = make_desc(b16 + j * 2048, BK * 128, 1024, LAYOUT_SW128);
            mma_f16(d_tmem, da, db, idesc, (kb | (uint32_t)j) != 0u);
          }
          tc_commit(empty(stage));
          if (kb + 1 == k_blocks) tc_commit(acc_full(buf));
        }
        __syncwarp();
        if (++stage == C::STAGES) { stage = 0; phase ^= 1u; }
      }
    }
  } else if (warp >= 6) {
    // ------------------------------------------------------------ f32 -> f16 converters
    // The raw tile is 1024 float4 (row r = f / 8, float4 c4 = f % 8); consecutive
    // threads take consecutive float4 (conflict-free reads) and each writes the 8
    // bytes of f16 it produced into 16-byte chunk (c4 / 2) ^ ((r >> 1) & 3) of
    // the row: the 64-byte swizzle the descriptor names.
    const int t = (threadIdx.x - 6 * 32) & 127, group = (threadIdx.x - 6 * 32) >> 7;
    uint32_t stage = 0, phase = 0, it_all = 0;
    bool ok = true;
    for (uint32_t tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x) {
      for (uint32_t kb = 0; kb < k_blocks; ++kb, ++it_all) {
        if ((int)(it_all % CVT_GROUPS) == group) {
          ok = mbar_wait(full_raw(stage), phase, abort_flag);
          if (!ok) break;
          const float4 *raw = reinterpret_cast<const float4 *>(smem_gen + stage * C::STAGE_BYTES);
          uint8_t *a16 = smem_gen + stage * C::STAGE_BYTES + C::RAW_BYTES;
          float4 v[(BM * BK / 4) / 128];
#pragma unroll
          for (int it = 0; it < (BM * BK / 4) / 128; ++it) v[it] = raw[t + it * 128];
#pragma unroll
          for (int it = 0; it < (BM * BK / 4) / 128; ++it) {
            const int f = t + it * 128;
            const int r = f >> 3, c4 = f & 7;
            const int chunk = (c4 >> 1) ^ ((r >> 1) & 3);
            uint2 h;
            h.x = pack_half2(v[it].x, v[it].y);
            h.y = pack_half2(v[it].z, v[it].w);
            *reinterpret_cast<uint2 *>(a16 + r * 64 + chunk * 16 + (c4 & 1) * 8) = h;
          }
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
          mbar_arrive(full_cvt(stage));
        }
        if (++stage == C::STAGES) { stage = 0; phase ^= 1u; }
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 0-3)
    uint32_t acc_it = 0;
    bool ok = true;
    const bool alpha_is_one = p.alpha == 1.0f;
    for (uint32_t tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x, ++acc_it) {
      const uint32_t batch = tile / tiles_per_batch, rem = tile % tiles_per_batch;
      const uint32_t m0 = (rem % tiles_m) * BM, n0 = (rem / tiles_m) * BN;
      const uint32_t buf = acc_it & 1u, acc_phase = (acc_it >> 1) & 1u;
      ok = mbar_wait(acc_full(buf), acc_phase, abort_flag, 256);
      if (!ok) break;
      tc_fence_after();
      const uint32_t row = m0 + warp * 32 + lane;
      const bool row_ok = row < p.m;
      const size_t row_off = (size_t)batch * p.stride_c + (size_t)row * p.n;
      float *__restrict__ crow = p.c + row_off;
      const float *__restrict__ drow = p.d ? p.d + row_off : nullptr;
      const float *__restrict__ bias = p.bias ? p.bias + (size_t)batch * p.bias_stride : nullptr;
      const uint32_t taddr = tmem_base + buf * BN + ((uint32_t)(warp * 32) << 16);
      epi_dispatch_act(p.act, [&](auto act_tag) {
        constexpr uint32_t ACT = decltype(act_tag)::value;
  #pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += 32) {
          float v[32];
          tmem_ld32(taddr + c0, v);
          const uint32_t col0 = n0 + c0;
          if (row_ok && col0 < p.n) {
  #pragma unroll
            for (int q = 0; q < 32; q += 4) {
              const uint32_t col = col0 + q;
              if (col < p.n) {  // N % 8 == 0: a float4 is either fully in or fully out
                float4 o = make_float4(v[q], v[q + 1], v[q + 2], v[q + 3]);
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
          }
        }
      });
      tc_fence_before();
      mbar_arrive(acc_empty(buf));
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
  if (warp == 5) {
    tc_fence_after();
    tmem_dealloc(tmem_base, C::TMEM_COLS);
  }
}

// ------------------------------------------------------------------ pre-converted A
// When the caller's slot has scratch for it, A is rounded to f16 once per launch by a small
// elementwise kernel (rows padded to a multiple of 8 halves) and the GEMM becomes a plain
// TMA -> tcgen05 pipeline: no converter warps, no raw f32 tile in shared memory, K blocks of 64.
// Both operands take the 128-byte swizzle (A K-major: SBO 1024; B N-major: LBO 64*128, SBO 1024).
constexpr int PK = 64;                       // K elements per stage
constexpr int PRE_THREADS = 192;             // warps 0-3 epilogue, 4 TMA, 5 MMA + TMEM
constexpr int EPI_PITCH = 36;                // floats per row of an epilogue transpose buffer

template <int BN>
struct PreCfg {
  static constexpr int A_BYTES = BM * PK * 2;             // 16 KiB
  static constexpr int B_BYTES = PK * BN * 2;             // 32 KiB at BN = 256
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES = (BN == 256) ? 4 : (BN == 192 ? 4 : (BN == 128 ? 6 : 8));
  // + per epilogue warp two 32 x 32 f32 blocks (4 KiB each, 1 KiB aligned): the sources of the TMA
  // stores of C in the 128-byte swizzle, or one transpose buffer of row pitch 36 floats
  static constexpr int EPI_BYTES = 4 * 2 * 4096;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + EPI_BYTES + 256 + 1024;
  static constexpr int ACC_STRIDE = BN == 192 ? 256 : BN;  // tensor-memory columns between the two accumulators
  static constexpr int TMEM_COLS = 2 * ACC_STRIDE;         // 128, 256 or 512: powers of two
};

__global__ void __launch_bounds__(256)
convert_a_f16_kernel(const float *__restrict__ a, __half *__restrict__ out, uint32_t k, uint32_t kp, uint64_t rows) {
  // one thread per 8 output halves (16 bytes); the pad columns k..kp-1 are zeros
  // chained launch: this kernel waits for the producer of A; the GEMM launched behind it may set
  // itself up while this one runs and waits for this grid to finish before it reads the copy
  TA_CHAIN_ENTER();
  const uint64_t idx = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const uint32_t per_row = kp / 8;
  if (idx >= rows * per_row) return;
  const uint64_t r = idx / per_row;
  const uint32_t c = (uint32_t)(idx % per_row) * 8;
  const float *src = a + r * k + c;
  float v[8];
  if (c + 8 <= k && (k & 3u) == 0) {
    const float4 x = *reinterpret_cast<const float4 *>(src), y = *reinterpret_cast<const float4 *>(src + 4);
    v[0] = x.x; v[1] = x.y; v[2] = x.z; v[3] = x.w; v[4] = y.x; v[5] = y.y; v[6] = y.z; v[7] = y.w;
  } else {
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = c + i < k ? src[i] : 0.0f;
  }
  uint4 o;
  o.x = pack_half2(v[0], v[1]); o.y = pack_half2(v[2], v[3]);
  o.z = pack_half2(v[4], v[5]); o.w = pack_half2(v[6], v[7]);
  *reinterpret_cast<uint4 *>(out + r * kp + c) = o;
}


// SPLITK: for problems whose tiles fill less than one wave of SMs.  A unit is (tile, K slice s of S);
// units = tiles * S is at most the SM count, so every unit has its own resident CTA.  Each CTA
// accumulates its K slice in tensor memory and stores the raw 128 x BN partial tile to scratch;
// when all S partials of a tile have arrived (a ticket per tile, bounded wait), each of the S CTAs
// adds the partials of ITS column slice of the tile in slice order and runs the epilogue on it.
// The order of the sum is fixed, so results are run-to-run bit-identical, and the reduction is
// spread over the CTAs that would otherwise idle.
template <int BN, bool SPLITK, bool DUAL = false>
__global__ void __launch_bounds__(PRE_THREADS, 1)
gemm_f16w_pre_kernel(const GemmParams p, const __grid_constant__ CUtensorMap map_a,
                     const __grid_constant__ CUtensorMap map_b, const __grid_constant__ CUtensorMap map_c,
                     const __grid_constant__ CUtensorMap map_b2, const __grid_constant__ CUtensorMap map_c2,
                     uint32_t *__restrict__ status) {
  static_assert(!DUAL || (!SPLITK && BN % 128 == 0), "the dual form takes whole 64-column groups of each matrix and no K split");
  // DUAL: a tile is BN / 2 output columns; the B stage holds those columns of b, then of b2
  constexpr int BNO = DUAL ? BN / 2 : BN;
  using C = PreCfg<BN>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t *smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t epi_base = smem_base + C::STAGES * C::STAGE_BYTES;      // 1 KiB aligned: stages are multiples of 1 KiB
  const uint32_t bar_base = epi_base + C::EPI_BYTES;
  auto full = [&](int s) { return bar_base + 8u * s; };
  auto empty = [&](int s) { return bar_base + 8u * (C::STAGES + s); };
  auto acc_full = [&](int b) { return bar_base + 8u * (2 * C::STAGES + b); };
  auto acc_empty = [&](int b) { return bar_base + 8u * (2 * C::STAGES + 2 + b); };
  volatile uint32_t *tmem_slot =
      reinterpret_cast<volatile uint32_t *>(smem_gen + C::STAGES * C::STAGE_BYTES + C::EPI_BYTES + 8 * (2 * C::STAGES + 4));
  volatile uint32_t *abort_flag = tmem_slot + 1;
  const uint32_t red_bar = bar_base + 8u * (2 * C::STAGES + 4) + 16u;   // the split reduce's bulk copies land on it
  float *epi_buf = reinterpret_cast<float *>(smem_gen + C::STAGES * C::STAGE_BYTES);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < C::STAGES; ++s) {
      mbar_init(full(s), 1);
      mbar_init(empty(s), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(acc_full(b), 1);
      mbar_init(acc_empty(b), 128);
    }
    mbar_init(red_bar, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 5) tmem_alloc(smem_u32((const void *)tmem_slot), C::TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // launched with programmatic stream serialization behind the conversion of A: barriers, tensor
  // memory and the tensor maps are set up by now; nothing below touches global memory before the
  // conversion kernel has finished
  if (p.pdl_wait) TA_CHAIN_ENTER();

  const uint32_t tiles_m = (p.m + BM - 1) / BM, tiles_n = (p.n + BNO - 1) / BNO;
  const uint32_t tiles_per_batch = tiles_m * tiles_n;
  const uint32_t splits = SPLITK ? p.fw_splits : 1u;
  const uint32_t num_tiles = tiles_per_batch * p.batch * splits;     // work units
  const uint32_t k_blocks_all = (p.k + PK - 1) / PK;
  // unit -> tile (batch, position), K slice and its K blocks [kb_lo, kb_hi): slices of one tile are
  // neighbouring units, so their CTAs run side by side
  auto decode = [&](uint32_t unit, uint32_t &tile_id, uint32_t &slice, uint32_t &kb_lo, uint32_t &kb_hi) {
    tile_id = unit / splits;
    slice = unit % splits;
    const uint32_t per = k_blocks_all / splits, rem = k_blocks_all % splits;
    kb_lo = slice * per + min(slice, rem);
    kb_hi = kb_lo + per + (slice < rem ? 1u : 0u);
  };

  if (warp == 4) {
    uint32_t stage = 0, phase = 0;
    bool ok = true;
    for (uint32_t unit = blockIdx.x; ok && unit < num_tiles; unit += gridDim.x) {
      uint32_t tile, slice, kb_lo, kb_hi;
      decode(unit, tile, slice, kb_lo, kb_hi);
      const uint32_t batch = tile / tiles_per_batch, rem = tile % tiles_per_batch;
      const int m0 = (int)(rem % tiles_m) * BM, n0 = (int)(rem / tiles_m) * BNO;
      const int za = p.stride_a ? (int)batch : 0, zb = p.stride_b ? (int)batch : 0;
      for (uint32_t kb = kb_lo; kb < kb_hi; ++kb) {
        ok = mbar_wait(empty(stage), phase ^ 1u, abort_flag);
        if (!ok) break;
        const uint32_t dst = smem_base + stage * C::STAGE_BYTES;
        if (elect_one()) {
          mbar_arrive_expect_tx(full(stage), C::STAGE_BYTES);
          tma_load_3d(dst, &map_a, full(stage), (int)(kb * PK), m0, za);
          if constexpr (DUAL) {   // grouped views only (N % 64 == 0): BN / 128 groups of each matrix
            tma_load_4d(dst + C::A_BYTES, &map_b, full(stage), 0, (int)(kb * PK), n0 / 64, zb);
            tma_load_4d(dst + C::A_BYTES + (BNO / 64) * (PK * 128), &map_b2, full(stage), 0, (int)(kb * PK), n0 / 64, zb);
          } else if (p.b_grouped) {
            tma_load_4d(dst + C::A_BYTES, &map_b, full(stage), 0, (int)(kb * PK), n0 / 64, zb);
          } else {
#pragma unroll
            for (int nb = 0; nb < BN / 64; ++nb)
              tma_load_3d(dst + C::A_BYTES + nb * (PK * 128), &map_b, full(stage), n0 + nb * 64, (int)(kb * PK), zb);
          }
        }
        __syncwarp();
        if (++stage == C::STAGES) { stage = 0; phase ^= 1u; }
      }
    }
  } else if (warp == 5) {
    const uint32_t idesc = (1u << 4) | (1u << 16) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
    uint32_t stage = 0, phase = 0, acc_it = 0;
    bool ok = true;
    for (uint32_t unit = blockIdx.x; ok && unit < num_tiles; unit += gridDim.x, ++acc_it) {
      uint32_t tile, slice, kb_lo, kb_hi;
      decode(unit, tile, slice, kb_lo, kb_hi);
      const uint32_t buf = acc_it & 1u, acc_phase = (acc_it >> 1) & 1u;
      ok = mbar_wait(acc_empty(buf), acc_phase ^ 1u, abort_flag);
      if (!ok) break;
      tc_fence_after();
      const uint32_t d_tmem = tmem_base + buf * C::ACC_STRIDE;
      for (uint32_t kb = kb_lo; kb < kb_hi; ++kb) {
        ok = mbar_wait(full(stage), phase, abort_flag);
        if (!ok) break;
        tc_fence_after();
        // descriptors are built warp-uniformly; advancing K by 16 halves moves A by 32 bytes
        // (+2 in the 16-byte address field) and MN-major B by 16 rows of 128 bytes (+128)
        const uint32_t a16 = smem_base + stage * C::STAGE_BYTES;
        const uint64_t da0 = make_desc(a16, 16, 1024, LAYOUT_SW128);
        const uint64_t db0 = make_desc(a16 + C::A_BYTES, PK * 128, 1024, LAYOUT_SW128);
        if (elect_one()) {
#pragma unroll
          for (int j = 0; j < PK / 16; ++j)
            mma_f16(d_tmem, da0 + (uint64_t)(j * 2), db0 + (uint64_t)(j * 128), idesc, ((kb - kb_lo) | (uint32_t)j) != 0u);
          tc_commit(empty(stage));
          if (kb + 1 == kb_hi) tc_commit(acc_full(buf));
        }
        __syncwarp();
        if (++stage == C::STAGES) { stage = 0; phase ^= 1u; }
      }
    }
  } else {
    uint32_t acc_it = 0;
    bool ok = true;
    const bool alpha_is_one = p.alpha == 1.0f;
    for (uint32_t unit = blockIdx.x; ok && unit < num_tiles; unit += gridDim.x, ++acc_it) {
      uint32_t tile, slice, kb_lo, kb_hi;
      decode(unit, tile, slice, kb_lo, kb_hi);
      const uint32_t batch = tile / tiles_per_batch, rem = tile % tiles_per_batch;
      const uint32_t m0 = (rem % tiles_m) * BM, n0 = (rem / tiles_m) * BNO;
      const uint32_t buf = acc_it & 1u, acc_phase = (acc_it >> 1) & 1u;
      ok = mbar_wait(acc_full(buf), acc_phase, abort_flag, 256);
      if (!ok) break;
      tc_fence_after();
      if constexpr (SPLITK) {
        // ---- raw partial tile to scratch in the accumulator's own layout: float4 column group g of row r
        // at part4[g * 128 + r].  A lane holds one row, so a warp's store covers 512 contiguous bytes
        // and nothing is transposed; the reducing pass below reads the same layout.
        float4 *__restrict__ part4 = reinterpret_cast<float4 *>(p.fw_partials + (size_t)unit * (BM * BN));
        const uint32_t taddr = tmem_base + buf * C::ACC_STRIDE + ((uint32_t)(warp * 32) << 16);
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += 32) {
          float v[32];
          tmem_ld32(taddr + c0, v);
#pragma unroll
          for (int q = 0; q < 8; ++q)
            part4[(size_t)(c0 / 4 + q) * BM + warp * 32 + lane] = make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
        }
        tc_fence_before();
        mbar_arrive(acc_empty(buf));
        // ---- ticket: wait (bounded) until every slice of this tile has stored its partial
        __threadfence();
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (threadIdx.x == 0) {
          atomicAdd(&p.fw_counters[2 * tile], 1u);
          const uint64_t t0 = global_timer_ns();
          uint32_t seen = 0, spins = 0;
          for (;;) {
            asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(seen) : "l"(p.fw_counters + 2 * tile) : "memory");
            if (seen >= splits) break;
            if ((++spins & 63u) == 0 && (*abort_flag || global_timer_ns() - t0 > WAIT_LIMIT_NS)) {
              *abort_flag = 1;
              break;
            }
          }
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (*abort_flag) { ok = false; break; }
        __threadfence();
        // ---- this CTA's column slice of the tile: add the S partials in slice order, epilogue, store.
        // In the partial layout the slice of one partial is contiguous (column groups x 128 rows x 16
        // bytes), so S bulk copies bring all of it into the idle pipeline stages in one round trip;
        // a lane then owns a row, reads conflict-free from shared memory and writes its 16-byte
        // pieces of C (the slice is 32 KiB per CTA: the row-strided stores are not what costs).
        const uint32_t g4n = BN / splits / 4;                   // float4 column groups of this CTA's slice (splits divides BN / 4)
        const uint32_t g4_base = slice * g4n;
        const uint32_t slice_bytes = g4n * BM * 16u;
        if (threadIdx.x == 0) {
          asm volatile("fence.proxy.async;" ::: "memory");     // the partials were written through the generic proxy
          mbar_arrive_expect_tx(red_bar, slice_bytes * splits);
          const uint8_t *src = reinterpret_cast<const uint8_t *>(p.fw_partials + (size_t)tile * splits * (BM * BN)) +
                               (size_t)g4_base * BM * 16u;
          for (uint32_t t = 0; t < splits; ++t)
            asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                         ::"r"(smem_base + t * slice_bytes), "l"(src + (size_t)t * (BM * BN * 4)), "r"(slice_bytes), "r"(red_bar)
                         : "memory");
        }
        ok = mbar_wait(red_bar, acc_it & 1u, abort_flag, 64);
        if (!ok) break;
        const float4 *__restrict__ sm4 = reinterpret_cast<const float4 *>(smem_gen);
        const size_t plane_off = (size_t)batch * p.stride_c;
        const float *__restrict__ bias = p.bias ? p.bias + (size_t)batch * p.bias_stride : nullptr;
        const uint32_t r = warp * 32 + lane, row = m0 + r;
        const bool row_ok = row < p.m;
        // blocks of 32 columns (8 float4 groups); a slice whose width is a multiple of 32 leaves
        // through TMA stores like the unsplit tile, any other one is stored by the lanes
        const bool tma_out = p.c_tma && (g4n % 8u) == 0;
        uint32_t blk = 0;
        epi_dispatch_act(p.act, [&](auto act_tag) {
          constexpr uint32_t ACT = decltype(act_tag)::value;
          constexpr uint32_t U = 8;
          for (uint32_t g0 = 0; g0 < g4n; g0 += U, ++blk) {
            float4 acc[U], c_old[U], dv[U], bv[U];
            bool live[U];
#pragma unroll
            for (uint32_t u = 0; u < U; ++u) {
              const uint32_t g4 = g0 + u, col = n0 + (g4_base + g4) * 4;
              live[u] = g4 < g4n && row_ok && col < p.n;
              c_old[u] = dv[u] = bv[u] = acc[u] = make_float4(0.f, 0.f, 0.f, 0.f);
              if (!live[u]) continue;
              const size_t off = plane_off + (size_t)row * p.n + col;
              if (p.accumulate) c_old[u] = *reinterpret_cast<const float4 *>(p.c + off);
              if (bias) bv[u] = __ldg(reinterpret_cast<const float4 *>(bias + col));
              if (p.d) dv[u] = *reinterpret_cast<const float4 *>(p.d + off);
            }
            for (uint32_t t = 0; t < splits; ++t) {
#pragma unroll
              for (uint32_t u = 0; u < U; ++u) {
                if (g0 + u >= g4n) continue;
                const float4 v = sm4[(size_t)t * (slice_bytes / 16u) + (size_t)(g0 + u) * BM + r];
                acc[u].x += v.x; acc[u].y += v.y; acc[u].z += v.z; acc[u].w += v.w;
              }
            }
#pragma unroll
            for (uint32_t u = 0; u < U; ++u) {
              float4 o = acc[u];
              if (!alpha_is_one) { o.x *= p.alpha; o.y *= p.alpha; o.z *= p.alpha; o.w *= p.alpha; }
              if (p.accumulate) { o.x += c_old[u].x; o.y += c_old[u].y; o.z += c_old[u].z; o.w += c_old[u].w; }
              o.x = epi_apply_t<ACT>(o.x, bias != nullptr, bv[u].x, p.binary, dv[u].x, p.beta);
              o.y = epi_apply_t<ACT>(o.y, bias != nullptr, bv[u].y, p.binary, dv[u].y, p.beta);
              o.z = epi_apply_t<ACT>(o.z, bias != nullptr, bv[u].z, p.binary, dv[u].z, p.beta);
              o.w = epi_apply_t<ACT>(o.w, bias != nullptr, bv[u].w, p.binary, dv[u].w, p.beta);
              acc[u] = o;
            }
            const uint32_t col0 = n0 + (g4_base + g0) * 4;
            if (tma_out) {
              if (col0 >= p.n) break;                      // warp-uniform
              const uint32_t sbuf = epi_base + (uint32_t)warp * 8192u + (blk & 1u) * 4096u;
              if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
              __syncwarp();
#pragma unroll
              for (uint32_t u = 0; u < U; ++u) {
                const uint32_t dst = sbuf + (uint32_t)lane * 128u + ((u ^ ((uint32_t)lane & 7u)) << 4);
                asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "f"(acc[u].x), "f"(acc[u].y), "f"(acc[u].z),
                             "f"(acc[u].w) : "memory");
              }
              asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
              __syncwarp();
              if (lane == 0) {
                asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%1, %2, %3}], [%4];" ::"l"(&map_c),
                             "r"((int)col0), "r"((int)(m0 + warp * 32)), "r"((int)batch), "r"(sbuf) : "memory");
                asm volatile("cp.async.bulk.commit_group;" ::: "memory");
              }
            } else {
#pragma unroll
              for (uint32_t u = 0; u < U; ++u)
                if (live[u]) *reinterpret_cast<float4 *>(p.c + plane_off + (size_t)row * p.n + col0 + 4 * u) = acc[u];
            }
          }
        });
        if (tma_out) {
          if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
          __syncwarp();
        }
        // ---- the last slice to finish reading puts the tile's two ticket words back to zero
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (threadIdx.x == 0) {
          if (atomicAdd(&p.fw_counters[2 * tile + 1], 1u) == splits - 1) {
            p.fw_counters[2 * tile] = 0u;
            p.fw_counters[2 * tile + 1] = 0u;
          }
        }
        continue;
      }
      if constexpr (DUAL) {
        // gate columns [0, BN/2) and up columns [BN/2, BN) of the accumulator: a lane reads its row of a
        // 32-column block of both, forms silu(gate) * up with the formulas of the separate epilogue
        // (activation, then the multiplying binary stage), and both blocks leave through TMA stores
        // (the product to C, the plain up values to C2): the warp's two staging buffers alternate
        const uint32_t taddr = tmem_base + buf * C::ACC_STRIDE + ((uint32_t)(warp * 32) << 16);
        const uint32_t sbuf0 = epi_base + (uint32_t)warp * 8192u, sbuf1 = sbuf0 + 4096u;
#pragma unroll 1
        for (int c0 = 0; c0 < BNO; c0 += 32) {
          if (n0 + c0 >= p.n) break;
          float g[32], u[32];
          tmem_ld32(taddr + c0, g);
          tmem_ld32(taddr + BNO + c0, u);
#pragma unroll
          for (int i = 0; i < 32; ++i)
            g[i] = epi_apply_t<(uint32_t)Activation::Silu>(g[i], false, 0.0f, (uint32_t)BinaryKind::Mul, u[i], 0.0f);
          // the product block of the chunk before must have been read (with C2 a second store is in flight)
          if (lane == 0) {
            if (p.c2) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
            else asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
          }
          __syncwarp();
#pragma unroll
          for (int q = 0; q < 8; ++q) {
            const uint32_t dst = sbuf0 + (uint32_t)lane * 128u + (((uint32_t)q ^ ((uint32_t)lane & 7u)) << 4);
            asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "f"(g[4 * q]), "f"(g[4 * q + 1]), "f"(g[4 * q + 2]),
                         "f"(g[4 * q + 3]) : "memory");
          }
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
          __syncwarp();
          if (lane == 0) {
            asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%1, %2, %3}], [%4];" ::"l"(&map_c),
                         "r"((int)(n0 + c0)), "r"((int)(m0 + warp * 32)), "r"((int)batch), "r"(sbuf0) : "memory");
            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
          }
          if (p.c2) {
            if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");   // the up block of the chunk before
            __syncwarp();
#pragma unroll
            for (int q = 0; q < 8; ++q) {
              const uint32_t dst = sbuf1 + (uint32_t)lane * 128u + (((uint32_t)q ^ ((uint32_t)lane & 7u)) << 4);
              asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "f"(u[4 * q]), "f"(u[4 * q + 1]), "f"(u[4 * q + 2]),
                           "f"(u[4 * q + 3]) : "memory");
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) {
              asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%1, %2, %3}], [%4];" ::"l"(&map_c2),
                           "r"((int)(n0 + c0)), "r"((int)(m0 + warp * 32)), "r"((int)batch), "r"(sbuf1) : "memory");
              asm volatile("cp.async.bulk.commit_group;" ::: "memory");
            }
          }
        }
        if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
        __syncwarp();
        tc_fence_before();
        mbar_arrive(acc_empty(buf));
        continue;
      }
      if (p.c_tma) {
        // C leaves through TMA: a lane holds one row of a 32 x 32 block, applies the epilogue to it
        // and writes it into a shared-memory block in the 128-byte swizzle (16-byte chunk c of row r
        // at chunk c ^ (r & 7): conflict-free); one lane then issues a bulk tensor store of the
        // block.  The stores are asynchronous: the warp goes on with the next block in its second
        // buffer and only waits, before reusing a buffer, until the store issued from it has READ it.
        // Rows and columns beyond M / N are clipped by the tensor map.  D and old C are read by
        // rows (16 bytes per lane and instruction; the eight instructions of a block use every
        // sector they touch).
        const size_t plane_off = (size_t)batch * p.stride_c;
        const float *__restrict__ bias = p.bias ? p.bias + (size_t)batch * p.bias_stride : nullptr;
        const uint32_t taddr = tmem_base + buf * C::ACC_STRIDE + ((uint32_t)(warp * 32) << 16);
        const uint32_t row = m0 + warp * 32 + lane;
        const bool row_ok = row < p.m;
        epi_dispatch_act(p.act, [&](auto act_tag) {
          constexpr uint32_t ACT = decltype(act_tag)::value;
          const bool plain = ACT == 0 && !bias && !p.d && !p.accumulate && alpha_is_one && p.binary == 0;
#pragma unroll 1
          for (int c0 = 0; c0 < BN; c0 += 32) {
            if (n0 + c0 >= p.n) break;
            const uint32_t sbuf = epi_base + (uint32_t)warp * 8192u + (uint32_t)((c0 >> 5) & 1) * 4096u;
            float v[32];
            tmem_ld32(taddr + c0, v);
            if (!plain) {
              float4 dv[8], co[8];
#pragma unroll
              for (int q = 0; q < 8; ++q) {
                dv[q] = co[q] = make_float4(0.f, 0.f, 0.f, 0.f);
                const uint32_t col = n0 + c0 + 4 * q;
                if (row_ok && col < p.n) {
                  const size_t off = plane_off + (size_t)row * p.n + col;
                  if (p.d) dv[q] = *reinterpret_cast<const float4 *>(p.d + off);
                  if (p.accumulate) co[q] = *reinterpret_cast<const float4 *>(p.c + off);
                }
              }
#pragma unroll
              for (int q = 0; q < 8; ++q) {
                const uint32_t col = n0 + c0 + 4 * q;
                float4 bv = make_float4(0.f, 0.f, 0.f, 0.f);
                if (bias && col < p.n) bv = __ldg(reinterpret_cast<const float4 *>(bias + col));
                float4 o = make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
                if (!alpha_is_one) { o.x *= p.alpha; o.y *= p.alpha; o.z *= p.alpha; o.w *= p.alpha; }
                if (p.accumulate) { o.x += co[q].x; o.y += co[q].y; o.z += co[q].z; o.w += co[q].w; }
                v[4 * q] = epi_apply_t<ACT>(o.x, bias != nullptr, bv.x, p.binary, dv[q].x, p.beta);
                v[4 * q + 1] = epi_apply_t<ACT>(o.y, bias != nullptr, bv.y, p.binary, dv[q].y, p.beta);
                v[4 * q + 2] = epi_apply_t<ACT>(o.z, bias != nullptr, bv.z, p.binary, dv[q].z, p.beta);
                v[4 * q + 3] = epi_apply_t<ACT>(o.w, bias != nullptr, bv.w, p.binary, dv[q].w, p.beta);
              }
            }
            // the store issued from this buffer two blocks ago must have read it
            if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
            __syncwarp();
#pragma unroll
            for (int q = 0; q < 8; ++q) {
              const uint32_t dst = sbuf + (uint32_t)lane * 128u + (((uint32_t)q ^ ((uint32_t)lane & 7u)) << 4);
              asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "f"(v[4 * q]), "f"(v[4 * q + 1]),
                           "f"(v[4 * q + 2]), "f"(v[4 * q + 3]) : "memory");
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) {
              asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%1, %2, %3}], [%4];" ::"l"(&map_c),
                           "r"((int)(n0 + c0)), "r"((int)(m0 + warp * 32)), "r"((int)batch), "r"(sbuf) : "memory");
              asm volatile("cp.async.bulk.commit_group;" ::: "memory");
            }
          }
        });
        if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");   // both buffers free for the next tile
        __syncwarp();
        tc_fence_before();
        mbar_arrive(acc_empty(buf));
        continue;
      }
      // TMEM gives each lane one row; a row-per-lane store would touch 32 rows per instruction.
      // Transpose 32 x 32 blocks through shared memory so that every global access of the
      // epilogue (C, D, the old C when accumulating) covers full 128-byte row segments.
      float *__restrict__ tbuf = epi_buf + warp * 2048;
      const uint32_t cq = (uint32_t)(lane & 7) * 4, rsub = (uint32_t)lane >> 3;
      const size_t plane_off = (size_t)batch * p.stride_c;
      const float *__restrict__ bias = p.bias ? p.bias + (size_t)batch * p.bias_stride : nullptr;
      const uint32_t taddr = tmem_base + buf * C::ACC_STRIDE + ((uint32_t)(warp * 32) << 16);
      // one dispatch on the activation per tile; the chunk loop below is compiled per activation
      epi_dispatch_act(p.act, [&](auto act_tag) {
        constexpr uint32_t ACT = decltype(act_tag)::value;
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += 32) {
          float v[32];
          tmem_ld32(taddr + c0, v);
#pragma unroll
          for (int q = 0; q < 32; q += 4)
            *reinterpret_cast<float4 *>(tbuf + lane * EPI_PITCH + q) = make_float4(v[q], v[q + 1], v[q + 2], v[q + 3]);
          __syncwarp();
          const uint32_t col = n0 + c0 + cq;
          if (col < p.n) {
            // One warp per scheduler runs this code, so nothing hides a dependent instruction's latency:
            // all loads of the chunk (shared-memory tile, D, old C) are issued first, the arithmetic
            // and the stores follow, and the loop-invariant cases are decided outside the row loop.
            float4 bv = make_float4(0.f, 0.f, 0.f, 0.f);
            if (bias) bv = __ldg(reinterpret_cast<const float4 *>(bias + col));
            float4 o[8], dv[8], c_old[8];
            const bool rows_all = m0 + warp * 32 + 32 <= p.m;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const uint32_t r = (uint32_t)i * 4 + rsub;
              o[i] = *reinterpret_cast<const float4 *>(tbuf + r * EPI_PITCH + cq);
              dv[i] = c_old[i] = make_float4(0.f, 0.f, 0.f, 0.f);
            }
            if (p.d) {
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                const uint32_t row = m0 + warp * 32 + (uint32_t)i * 4 + rsub;
                if (rows_all || row < p.m) dv[i] = *reinterpret_cast<const float4 *>(p.d + plane_off + (size_t)row * p.n + col);
              }
            }
            if (p.accumulate) {
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                const uint32_t row = m0 + warp * 32 + (uint32_t)i * 4 + rsub;
                if (!(rows_all || row < p.m)) continue;
                const size_t off = plane_off + (size_t)row * p.n + col;
                if (p.c_f16) {
                  const uint2 raw = *reinterpret_cast<const uint2 *>(reinterpret_cast<const __half *>(p.c) + off);
                  const float2 lo = __half22float2(*reinterpret_cast<const __half2 *>(&raw.x));
                  const float2 hi = __half22float2(*reinterpret_cast<const __half2 *>(&raw.y));
                  c_old[i] = make_float4(lo.x, lo.y, hi.x, hi.y);
                } else {
                  c_old[i] = *reinterpret_cast<const float4 *>(p.c + off);
                }
              }
            }
            const bool plain = ACT == 0 && !bias && !p.d && !p.accumulate && alpha_is_one && p.binary == 0;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const uint32_t row = m0 + warp * 32 + (uint32_t)i * 4 + rsub;
              if (!(rows_all || row < p.m)) continue;
              const size_t off = plane_off + (size_t)row * p.n + col;
              float4 v = o[i];
              if (!plain) {
                if (!alpha_is_one) { v.x *= p.alpha; v.y *= p.alpha; v.z *= p.alpha; v.w *= p.alpha; }
                if (p.accumulate) { v.x += c_old[i].x; v.y += c_old[i].y; v.z += c_old[i].z; v.w += c_old[i].w; }
                v.x = epi_apply_t<ACT>(v.x, bias != nullptr, bv.x, p.binary, dv[i].x, p.beta);
                v.y = epi_apply_t<ACT>(v.y, bias != nullptr, bv.y, p.binary, dv[i].y, p.beta);
                v.z = epi_apply_t<ACT>(v.z, bias != nullptr, bv.z, p.binary, dv[i].z, p.beta);
                v.w = epi_apply_t<ACT>(v.w, bias != nullptr, bv.w, p.binary, dv[i].w, p.beta);
              }
              if (p.c_f16) {
                const __half2 lo = __floats2half2_rn(v.x, v.y), hi = __floats2half2_rn(v.z, v.w);
                uint2 raw;
                raw.x = *reinterpret_cast<const uint32_t *>(&lo);
                raw.y = *reinterpret_cast<const uint32_t *>(&hi);
                *reinterpret_cast<uint2 *>(reinterpret_cast<__half *>(p.c) + off) = raw;
              } else {
                *reinterpret_cast<float4 *>(p.c + off) = v;
              }
            }
          }
          __syncwarp();
        }
      });
      tc_fence_before();
      mbar_arrive(acc_empty(buf));
    }
  }

  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    for (int i = 0; i < 64; ++i) __nanosleep(100000);
    if (threadIdx.x == 0) atomicOr(status, 1u);
    __syncthreads();
  }
  if (warp == 5) {
    tc_fence_after();
    tmem_dealloc(tmem_base, C::TMEM_COLS);
  }
}

template <int BN, bool SPLITK = false, bool DUAL = false>
void launch_pre_t(const Context &ctx, const GemmParams &p, __half *a16, uint32_t kp, uint32_t *status,
                  bool a16_ready, cudaStream_t stream) {
  using C = PreCfg<BN>;
  static bool attr_set[64] = {};
  if (!attr_set[ctx.device & 63]) {
    TA_CUDA(cudaFuncSetAttribute(gemm_f16w_pre_kernel<BN, SPLITK, DUAL>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES));
    attr_set[ctx.device & 63] = true;
  }
  const uint64_t ba = p.stride_a ? p.batch : 1, bb = p.stride_b ? p.batch : 1;
  const uint64_t rows = ba * p.m;
  const uint64_t items = rows * (kp / 8);
  CUtensorMap map_a, map_b, map_c, map_b2, map_c2;
  // A16 [ba, M, Kp] f16: 128-byte rows of 64 halves, 128-byte swizzle; columns >= K read as zero (TMA bound K)
  encode_map3(ctx, &map_a, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, a16, p.k, p.m, ba, (uint64_t)kp * 2,
              (uint64_t)p.m * kp * 2, PK, BM, CU_TENSOR_MAP_SWIZZLE_128B);
  const uint64_t b_batch_bytes = p.stride_b ? (uint64_t)p.stride_b * 2 : (uint64_t)p.k * p.n * 2;
  GemmParams pg = p;
  pg.b_grouped = p.n % 64 == 0 ? 1u : 0u;
  constexpr int BNO = DUAL ? BN / 2 : BN;      // output columns per tile
  if (DUAL) {         // BN / 128 column groups of each of the two matrices per stage
    if (!pg.b_grouped || !p.b2) fail("internal: dual f16w GEMM launched without a second matrix or with N %% 64 != 0");
    encode_map_grouped(ctx, &map_b, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, p.b, 2, p.n, p.k, bb, b_batch_bytes, 64, PK,
                       BNO / 64, CU_TENSOR_MAP_SWIZZLE_128B);
    encode_map_grouped(ctx, &map_b2, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, p.b2, 2, p.n, p.k, bb, b_batch_bytes, 64, PK,
                       BNO / 64, CU_TENSOR_MAP_SWIZZLE_128B);
  } else if (pg.b_grouped)   // one TMA per stage for the whole BN-wide B block
    encode_map_grouped(ctx, &map_b, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, p.b, 2, p.n, p.k, bb, b_batch_bytes, 64, PK,
                       BN / 64, CU_TENSOR_MAP_SWIZZLE_128B);
  else
    encode_map3(ctx, &map_b, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, p.b, p.n, p.k, bb, (uint64_t)p.n * 2, b_batch_bytes, 64, PK,
                CU_TENSOR_MAP_SWIZZLE_128B);
  // C [batch, M, N] f32 leaves through TMA stores of 32 x 32 blocks (128-byte rows, 128-byte swizzle)
  // when it is f32 and addressable by a tensor map; the kernel otherwise stores it itself
  pg.c_tma = (!p.c_f16 && p.n % 4 == 0 && (reinterpret_cast<uintptr_t>(p.c) & 15u) == 0 &&
              (p.stride_c % 4) == 0 && tunables().f16w_tma_store) ? 1u : 0u;
  if (pg.c_tma)
    encode_map3(ctx, &map_c, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, p.c, p.n, p.m, p.batch, (uint64_t)p.n * 4,
                p.stride_c ? (uint64_t)p.stride_c * 4 : (uint64_t)p.m * p.n * 4, 32, 32, CU_TENSOR_MAP_SWIZZLE_128B);
  else
    map_c = map_a;
  if (!DUAL) map_b2 = map_b;
  map_c2 = map_c;
  if (DUAL) {
    if (!pg.c_tma) fail("internal: dual f16w GEMM needs a TMA-addressable f32 C");
    if (p.c2)
      encode_map3(ctx, &map_c2, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, p.c2, p.n, p.m, p.batch, (uint64_t)p.n * 4,
                  p.stride_c ? (uint64_t)p.stride_c * 4 : (uint64_t)p.m * p.n * 4, 32, 32, CU_TENSOR_MAP_SWIZZLE_128B);
  }
  const uint64_t tiles = (uint64_t)((p.m + BM - 1) / BM) * ((p.n + BNO - 1) / BNO) * p.batch * (SPLITK ? p.fw_splits : 1u);
  if (SPLITK && tiles > (uint64_t)ctx.sm_count) fail("internal: split-K units (%llu) exceed the SM count", (unsigned long long)tiles);
  const uint32_t grid = (uint32_t)std::min<uint64_t>(tiles, (uint64_t)ctx.sm_count);
  // the conversion is launched only now, with the tensor maps encoded: the two launches reach the
  // device back to back, so the device does not idle between them while the host encodes
  if (!a16_ready) {
    launch_chained(convert_a_f16_kernel, dim3((unsigned)((items + 255) / 256)), dim3(256), 0, stream,
                   static_cast<const float *>(p.a), a16, p.k, kp, rows);
    g_launches.fetch_add(1, std::memory_order_relaxed);
  }
  // chained launch (right behind the conversion kernel, or behind whatever produced the operands):
  // start early, wait on the device (see the kernel)
  pg.pdl_wait = tunables().pdl ? 1u : 0u;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid, 1, 1);
  cfg.blockDim = dim3(PRE_THREADS, 1, 1);
  cfg.dynamicSmemBytes = C::SMEM_BYTES;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pg.pdl_wait ? 1 : 0;
  TA_CUDA(cudaLaunchKernelEx(&cfg, gemm_f16w_pre_kernel<BN, SPLITK, DUAL>, pg, map_a, map_b, map_c, map_b2, map_c2, status));
  g_launches.fetch_add(1, std::memory_order_relaxed);
}

template <int BN>
void launch_t(const Context &ctx, const GemmParams &p, uint32_t *status, cudaStream_t stream) {
  using C = Cfg<BN>;
  static bool attr_set[64] = {};
  if (!attr_set[ctx.device & 63]) {
    TA_CUDA(cudaFuncSetAttribute(gemm_f16w_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 C::SMEM_BYTES));
    attr_set[ctx.device & 63] = true;
  }
  CUtensorMap map_a, map_b;
  const uint64_t ba = p.stride_a ? p.batch : 1, bb = p.stride_b ? p.batch : 1;
  // A [ba, M, K] f32: plain 128-byte rows of 32 floats
  encode_map3(ctx, &map_a, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, p.a, p.k, p.m, ba, (uint64_t)p.k * 4,
              p.stride_a ? (uint64_t)p.stride_a * 4 : (uint64_t)p.m * p.k * 4, BK, BM,
              CU_TENSOR_MAP_SWIZZLE_NONE);
  // B [bb, K, N] f16: boxes of 64 columns (128 bytes) x BK rows, 128-byte swizzle
  encode_map3(ctx, &map_b, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, p.b, p.n, p.k, bb, (uint64_t)p.n * 2,
              p.stride_b ? (uint64_t)p.stride_b * 2 : (uint64_t)p.k * p.n * 2, 64, BK,
              CU_TENSOR_MAP_SWIZZLE_128B);
  const uint64_t tiles = (uint64_t)((p.m + BM - 1) / BM) * ((p.n + BN - 1) / BN) * p.batch;
  const uint32_t grid = (uint32_t)std::min<uint64_t>(tiles, (uint64_t)ctx.sm_count);
  gemm_f16w_kernel<BN><<<grid, NUM_THREADS, C::SMEM_BYTES, stream>>>(p, map_a, map_b, status);
  TA_CUDA(cudaGetLastError());
  g_launches.fetch_add(1, std::memory_order_relaxed);
}

}  // namespace

// TMA needs 16-byte strides and bases: K % 4 == 0 for the f32 A rows, N % 8 == 0
// for the f16 B rows; float4 epilogue accesses need N % 4 == 0 and aligned C/D/bias.
bool gemm_f16w_umma_eligible(const GemmParams &p) {
  if (!p.b_f16) return false;
  if (p.k % 4 || p.n % 8) return false;
  if ((reinterpret_cast<uintptr_t>(p.a) | reinterpret_cast<uintptr_t>(p.b) |
       reinterpret_cast<uintptr_t>(p.c)) & 15)
    return false;
  if (p.d && (reinterpret_cast<uintptr_t>(p.d) & 15)) return false;
  if (p.bias && (reinterpret_cast<uintptr_t>(p.bias) & 15)) return false;
  if ((p.stride_a % 4) || (p.stride_b % 8) || (p.stride_c % 4) || (p.bias_stride % 4)) return false;
  return true;
}

// Column-tile width: fewest waves of (tile width + fixed per-tile cost); the fixed
// part stands for the A staging and conversion every tile repeats.
uint32_t gemm_f16w_umma_tile_n(uint32_t batch, uint32_t m, uint32_t n, int sm_count) {
  uint32_t best = 256;
  uint64_t best_cost = ~0ull;
  for (uint32_t bn : {256u, 128u, 64u}) {
    const uint64_t tiles = (uint64_t)batch * ((m + BM - 1) / BM) * ((n + bn - 1) / bn);
    const uint64_t waves = (tiles + sm_count - 1) / sm_count;
    const uint64_t cost = waves * (bn + 96);
    if (cost < best_cost) {
      best_cost = cost;
      best = bn;
    }
  }
  return best;
}

// Row pitch (in halves) of the f16 copy of A: K rounded up to 8, plus the experiment switch f16w_apad.
static uint32_t a16_pitch(uint32_t k) { return ((k + 7u) & ~7u) + tunables().f16w_apad; }

uint32_t gemm_f16w_umma_a16_pitch(uint32_t k) { return a16_pitch(k); }

// Scratch bytes for the f16 copy of A (rounded up to 256) ...
static size_t a16_bytes(uint32_t batch_a, uint32_t m, uint32_t k) {
  return ((size_t)((uint64_t)batch_a * m * a16_pitch(k) * 2) + 255u) & ~(size_t)255u;
}
size_t gemm_f16w_umma_scratch_bytes(uint32_t batch_a, uint32_t m, uint32_t k) { return a16_bytes(batch_a, m, k); }

// Tile width and K split for a problem on the pre-converted-A kernel.  The 512-row prefill shapes
// have 32..176 tiles for 148 SMs and a CTA takes in about 130 GB/s of operands, so what a CTA moves
// decides the time: cost = K blocks per CTA x KiB per block (A 16 + B BN / 8), plus a fixed charge
// for the split's partial-tile round trip.  Measured over tile widths and splits on 512 x {2048,
// 2560, 5632} x 2048, 512 x 2048 x 5632 and 1024 x 4096 x 1024: time = 17 us + 7.6 ns per KiB, a
// split adds 4.5 to 6 us (650 KiB-equivalents).  Units (tiles x splits) must not exceed the SM count
// when splitting; several waves without a split are charged in full.
F16wPlan gemm_f16w_umma_plan(uint32_t batch, uint32_t m, uint32_t n, uint32_t k, int sm_count, bool allow_split) {
  F16wPlan best;
  double best_cost = 1e300;
  const uint32_t kb = (k + PK - 1) / PK;
  const int force = tunables().f16w_splitk;
  const uint32_t force_bn = tunables().f16w_bn;
  for (uint32_t bn : {256u, 192u, 128u, 64u}) {
    if (force_bn && bn != force_bn) continue;
    const uint64_t tiles = (uint64_t)batch * ((m + BM - 1) / BM) * ((n + bn - 1) / bn);
    const double block_kb = 16.0 + bn * 0.125;
    for (uint32_t s : {1u, 2u, 3u, 4u, 6u, 8u}) {
      if (s > 1 && (!allow_split || force == 0 || force == 1)) break;
      if (s > 1 && (tiles * s > (uint64_t)sm_count || kb / s < 4 || (bn / 4) % s != 0)) continue;
      if (force > 1 && s != (uint32_t)force && tiles * (uint64_t)force <= (uint64_t)sm_count && kb / force >= 4 && (bn / 4) % force == 0) continue;
      const uint64_t waves = s > 1 ? 1 : (tiles + sm_count - 1) / sm_count;
      const double cost = (double)waves * ((kb + s - 1) / s) * block_kb + (s > 1 ? 650.0 : 0.0) + 90.0 +
                          (bn == 192 && n % 192 ? 8.0 : 0.0);   // a partial last tile wastes part of its columns
      if (cost < best_cost) {
        best_cost = cost;
        best.tile_n = bn;
        best.splits = s;
      }
    }
  }
  best.partial_bytes = best.splits > 1
                           ? (size_t)batch * ((m + BM - 1) / BM) * ((n + best.tile_n - 1) / best.tile_n) * best.splits * BM * best.tile_n * 4
                           : 0;
  return best;
}

size_t gemm_f16w_umma_scratch_bytes_split(uint32_t batch, uint32_t batch_a, uint32_t m, uint32_t n, uint32_t k, int sm_count) {
  const F16wPlan plan = gemm_f16w_umma_plan(batch, m, n, k, sm_count, true);
  return a16_bytes(batch_a, m, k) + plan.partial_bytes;
}

// The SwiGLU pair as one launch: plain products (alpha 1, no bias / accumulate / D), f32 C and C2,
// one matrix per call, N a multiple of 64 (grouped weight views), everything 16-byte aligned, and
// the tunables that give the pre-converted-A kernel with TMA stores.
bool gemm_f16w_umma_dual_eligible(const GemmParams &p) {
  if (!gemm_f16w_umma_eligible(p) || !p.b2 || p.batch != 1 || p.n % 64 || p.c_f16) return false;
  if (p.alpha != 1.0f || p.accumulate || p.bias) return false;
  if ((reinterpret_cast<uintptr_t>(p.b2) | reinterpret_cast<uintptr_t>(p.c) | reinterpret_cast<uintptr_t>(p.c2)) & 15u) return false;
  return tunables().f16w_pre && tunables().f16w_tma_store && tunables().f16w_dual;
}

void launch_gemm_f16w_umma_dual(const Context &ctx, const GemmParams &p, uint32_t *status, void *scratch, size_t scratch_bytes,
                                bool a16_ready, cudaStream_t stream) {
  if (!gemm_f16w_umma_dual_eligible(p)) fail("internal: dual f16w GEMM launched on an ineligible problem");
  if (!scratch || scratch_bytes < gemm_f16w_umma_scratch_bytes(1, p.m, p.k) || (reinterpret_cast<uintptr_t>(scratch) & 15u))
    fail("internal: dual f16w GEMM needs scratch for the f16 copy of A");
  launch_pre_t<256, false, true>(ctx, p, static_cast<__half *>(scratch), a16_pitch(p.k), status, a16_ready, stream);
}

void launch_gemm_a16_umma(const Context &ctx, const GemmParams &p_in, uint32_t tile_n, uint32_t *status,
                          cudaStream_t stream) {
  if (!p_in.b_f16 || p_in.k % 8 || p_in.n % 8)
    fail("a16 tensor-core GEMM needs f16 A, B and C with K and N multiples of 8");
  if ((reinterpret_cast<uintptr_t>(p_in.a) | reinterpret_cast<uintptr_t>(p_in.b) | reinterpret_cast<uintptr_t>(p_in.c)) & 15)
    fail("a16 tensor-core GEMM needs 16-byte aligned operands");
  if (p_in.stride_a % 8) fail("a16 tensor-core GEMM needs an A batch stride that is a multiple of 8 halves");
  GemmParams p = p_in;
  p.c_f16 = 1;
  __half *a16 = static_cast<__half *>(const_cast<void *>(p.a));   // A as stored: [batch, M, K] halves, pitch K
  if (tile_n >= 256) launch_pre_t<256>(ctx, p, a16, p.k, status, true, stream);
  else if (tile_n >= 128) launch_pre_t<128>(ctx, p, a16, p.k, status, true, stream);
  else launch_pre_t<64>(ctx, p, a16, p.k, status, true, stream);
}

void launch_gemm_f16w_umma(const Context &ctx, const GemmParams &p_in, uint32_t tile_n, uint32_t *status,
                           void *scratch, size_t scratch_bytes, bool a16_ready, cudaStream_t stream,
                           uint32_t *counters, bool auto_plan) {
  if (!gemm_f16w_umma_eligible(p_in))
    fail("f16w tensor-core GEMM needs f32 A, f16 B, K %% 4 == 0 and N %% 8 == 0");
  const uint32_t batch_a = p_in.stride_a ? p_in.batch : 1;
  if (scratch && scratch_bytes >= gemm_f16w_umma_scratch_bytes(batch_a, p_in.m, p_in.k) &&
      (reinterpret_cast<uintptr_t>(scratch) & 15u) == 0 && tunables().f16w_pre) {
    const uint32_t kp = a16_pitch(p_in.k);
    __half *a16 = static_cast<__half *>(scratch);
    GemmParams p = p_in;
    if (auto_plan) {
      // the routing heuristic's call: tile width and K split chosen together for this shape
      const F16wPlan plan = gemm_f16w_umma_plan(p.batch, p.m, p.n, p.k, ctx.sm_count, counters != nullptr);
      const size_t a16b = a16_bytes(batch_a, p.m, p.k);
      if (plan.splits > 1 && counters && scratch_bytes >= a16b + plan.partial_bytes) {
        p.fw_splits = plan.splits;
        p.fw_partials = reinterpret_cast<float *>(static_cast<uint8_t *>(scratch) + a16b);
        p.fw_counters = counters + F16W_SPLIT_COUNTER0;
        if (plan.tile_n == 256) launch_pre_t<256, true>(ctx, p, a16, kp, status, a16_ready, stream);
        else if (plan.tile_n == 192) launch_pre_t<192, true>(ctx, p, a16, kp, status, a16_ready, stream);
        else if (plan.tile_n == 128) launch_pre_t<128, true>(ctx, p, a16, kp, status, a16_ready, stream);
        else launch_pre_t<64, true>(ctx, p, a16, kp, status, a16_ready, stream);
        return;
      }
      const F16wPlan whole = plan.splits > 1 ? gemm_f16w_umma_plan(p.batch, p.m, p.n, p.k, ctx.sm_count, false) : plan;
      tile_n = whole.tile_n;
    }
    if (tile_n >= 256) launch_pre_t<256>(ctx, p, a16, kp, status, a16_ready, stream);
    else if (tile_n == 192) launch_pre_t<192>(ctx, p, a16, kp, status, a16_ready, stream);
    else if (tile_n >= 128) launch_pre_t<128>(ctx, p, a16, kp, status, a16_ready, stream);
    else launch_pre_t<64>(ctx, p, a16, kp, status, a16_ready, stream);
    return;
  }
  const GemmParams &p = p_in;
  if (tile_n >= 256) launch_t<256>(ctx, p, status, stream);
  else if (tile_n >= 128) launch_t<128>(ctx, p, status, stream);
  else launch_t<64>(ctx, p, status, stream);
}

}  // namespace ta
