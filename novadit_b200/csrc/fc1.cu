// Fused FC1: y = epilogue((x @ w^T) * alpha + bias) on the 5th-generation tensor cores (sm_100a).
//
// One persistent CTA per SM, 320 threads, warp-specialised:
//   warp 0      TMA producer (one thread): x and w tiles -> 128B-swizzled shared memory, mbarrier ring
//   warp 1      tcgen05.mma issuer (one thread) + owner of the tensor-memory allocation
//   warps 2..9  epilogue (two warps per TMEM lane quarter, each taking half of the tile's columns):
//               tcgen05.ld the fp32 accumulator, * alpha, + bias, activation (gated: value * act(gate)), round
//               once, stage a 32 x 32 block in shared memory and hand it to the copy engine (bulk tensor store)
// CTA tile: 128 rows x 256 accumulator columns x 128 bytes of K per stage. For the gated form
// the 256 columns are 128 gate columns and the 128 value columns of the SAME output columns,
// staged as one K-major B operand (gate rows then value rows), so a single UMMA of N=256
// produces both halves and the epilogue combines TMEM columns c and 128+c. Two accumulators
// (2 x 256 of the 512 TMEM columns) let the epilogue of tile i overlap the main loop of tile i+1.
//
// Three kernels share these pieces:
//   fc1_kernel          single-CTA tiles (cta_group::1), 4 operand stages
//   fc1_pair_kernel     two-CTA tiles (cta_group::2, clusters of two): 256 x 256 per pair, each CTA stages its A
//                       rows and half of B, one MMA stream for both tensor cores; no multicast loads
//   fc1_kernel<BWD>     the backward-dz variant: the same main loop (3 stages) with the activation BACKWARD as
//                       epilogue - dy fetched by the copy engine, the two halves of dz stored as blocks
//
// Every wait on an mbarrier is bounded (1 s of %globaltimer); on expiry the waiting role raises
// a CTA-wide abort flag, the caller's status word and the device error word are set, every role leaves its loop,
// the producer lets its copies in flight land, and tensor memory is freed before the CTA exits.
#include <cuda.h>
#include <cuda_fp8.h>

#include <atomic>
#include <mutex>

#include "common.cuh"
#include "ptx.cuh"

namespace nd {

constexpr int kBM = 128;         // rows per CTA tile
constexpr int kBN = 256;         // accumulator columns per CTA tile
constexpr int kBKBytes = 128;    // bytes of K per stage = one 128B swizzle span
constexpr int kStages = 4;
constexpr int kEpilogueWarps = 8;
constexpr int kThreads = 64 + 32 * kEpilogueWarps;
constexpr int kATileBytes = kBM * kBKBytes;          // 16 KB
constexpr int kBHalfBytes = 128 * kBKBytes;          // 16 KB (128 weight rows)
constexpr int kStageBytes = kATileBytes + 2 * kBHalfBytes;  // 48 KB
constexpr int kTmemCols = 512;
constexpr int kOutBlockBytes = 32 * 32 * 2;  // 32 rows x 32 output columns of a 16-bit type
constexpr int kGroupM = 8;       // tile rasterisation: m-blocks per group
constexpr unsigned long long kWaitLimitNs = 1000000000ull;

// Where an expired wait is recorded: the caller's status word (nullable) and the device error word that
// nd_device_error() reads (codes 101.. there, so that they cannot be mistaken for the norm kernels' 1..3).
struct Fc1Sink {
  int* status;
  int* err;
};

struct Fc1Args {
  const void* bias;        // out dtype, length n (nullable)
  void* y;
  const float* alpha_dev;  // nullable, two floats multiplied into alpha
  Fc1Sink sink;
  long long* trace;        // nullable: per-role cycle counters (see nd_tune_fc1_trace)
  float* dbias_part;       // nullable (backward only): [tiles_m * 4][n] column sums of dz per 32-row quarter
  float alpha_host;
  int m, k, n;             // n = rows of w
  int n_out;               // columns of y (n/2 gated, n plain)
  int tiles_m, tiles_n, k_blocks;
};

constexpr int kBwdStages = 3;  // the backward-dz variant trades one operand stage for two more epilogue blocks

// STAGES operand stages; BLOCKS 32 x 32 staging blocks per epilogue warp (1: output; 3: dy in, two dz halves out)
template <int STAGES, int BLOCKS>
struct __align__(1024) Fc1SmemT {
  uint8_t stage[STAGES][kStageBytes];
  uint8_t out[kEpilogueWarps][BLOCKS][kOutBlockBytes];  // staging, private to each epilogue warp
  alignas(16) float bias[kEpilogueWarps][kBN];  // one private copy per epilogue warp: no cross-warp barrier in the epilogue
  uint64_t full[STAGES];
  uint64_t empty[STAGES];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint64_t dy_full[kEpilogueWarps];  // backward: the warp's dy block has landed
  uint32_t tmem_base;
  int abort_flag;
};
using Fc1Smem = Fc1SmemT<kStages, 1>;
using Fc1BwdSmem = Fc1SmemT<kBwdStages, 3>;

// Bounded wait. Returns false if the CTA is aborting or the limit expired (and raises the abort).
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag,
                                          Fc1Sink sink, int code) {
  if (mbar_try_wait(bar, parity)) return true;
  const unsigned long long t0 = global_ns();
  for (uint32_t polls = 1;; ++polls) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((polls & 255u) == 0) {
      if (*abort_flag) return false;
      if (global_ns() - t0 > kWaitLimitNs) {
        *abort_flag = 1;
        if (sink.status != nullptr) atomicCAS(sink.status, 0, code);
        if (sink.err != nullptr) atomicCAS(sink.err, 0, 100 + code);
        return false;
      }
    }
  }
}

// mbar_wait that also adds the cycles spent waiting to a per-role counter (lane 0 only; `acc` may be null)
__device__ __forceinline__ bool mbar_wait_timed(uint64_t* bar, uint32_t parity, volatile int* abort_flag, Fc1Sink sink,
                                                int code, long long* acc) {
  if (acc == nullptr) return mbar_wait(bar, parity, abort_flag, sink, code);
  const long long t0 = clock64();
  const bool ok = mbar_wait(bar, parity, abort_flag, sink, code);
  *acc += clock64() - t0;
  return ok;
}

__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, uint64_t* bar, int c0,
                                            int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(c0), "r"(c1)
      : "memory");
}

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tc_ld32(uint32_t taddr, float (&r)[32]) {
  uint32_t* u = reinterpret_cast<uint32_t*>(r);
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(u[0]), "=r"(u[1]), "=r"(u[2]), "=r"(u[3]), "=r"(u[4]), "=r"(u[5]), "=r"(u[6]), "=r"(u[7]),
        "=r"(u[8]), "=r"(u[9]), "=r"(u[10]), "=r"(u[11]), "=r"(u[12]), "=r"(u[13]), "=r"(u[14]),
        "=r"(u[15]), "=r"(u[16]), "=r"(u[17]), "=r"(u[18]), "=r"(u[19]), "=r"(u[20]), "=r"(u[21]),
        "=r"(u[22]), "=r"(u[23]), "=r"(u[24]), "=r"(u[25]), "=r"(u[26]), "=r"(u[27]), "=r"(u[28]),
        "=r"(u[29]), "=r"(u[30]), "=r"(u[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// K-major, 128B-swizzled operand tile: rows of 128 bytes, 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);  // start address, 16-byte units
  d |= static_cast<uint64_t>(1) << 16;                      // leading byte offset (unused for this layout)
  d |= static_cast<uint64_t>(1024 >> 4) << 32;              // stride byte offset between 8-row groups
  d |= static_cast<uint64_t>(1) << 46;                      // descriptor version of sm_100
  d |= static_cast<uint64_t>(2) << 61;                      // SWIZZLE_128B
  return d;
}

// dense MMA, fp32 accumulator, both operands K-major, M = 128, N = 256
__host__ __device__ constexpr uint32_t umma_idesc(uint32_t ab_format) {
  return (1u << 4) | (ab_format << 7) | (ab_format << 10) | ((kBN >> 3) << 17) | ((kBM >> 4) << 24);
}

__device__ __forceinline__ void tile_coords(const Fc1Args& a, int t, int& mi, int& ni) {
  const int per_group = kGroupM * a.tiles_n;
  const int g = t / per_group;
  const int first_m = g * kGroupM;
  const int gm = (a.tiles_m - first_m) < kGroupM ? (a.tiles_m - first_m) : kGroupM;
  const int r = t - g * per_group;
  mi = first_m + r % gm;
  ni = r / gm;
}

template <typename OUT> __device__ __forceinline__ uint32_t pack2(float a, float b);
template <> __device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float a, float b) {
  __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}
template <> __device__ __forceinline__ uint32_t pack2<__half>(float a, float b) {
  __half2 v = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}

template <typename OUT> __device__ __forceinline__ float2 unpack_pair(uint32_t w);
template <> __device__ __forceinline__ float2 unpack_pair<__nv_bfloat16>(uint32_t w) {
  return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xffff0000u));
}
template <> __device__ __forceinline__ float2 unpack_pair<__half>(uint32_t w) {
  return __half22float2(*reinterpret_cast<const __half2*>(&w));
}

// Bias of the tile's 256 accumulator columns -> one epilogue warp's shared-memory copy (fp32).
template <int GATED, typename OUT>
__device__ __forceinline__ void stage_bias(const Fc1Args& a, float* sb, int ni, int lane) {
  const OUT* __restrict__ bias = static_cast<const OUT*>(a.bias);
  const int out0 = GATED != 0 ? ni * 128 : ni * kBN;
#pragma unroll
  for (int h = 0; h < kBN / 32; ++h) {
    const int c = lane + h * 32;
    int wrow;  // row of w (= index into bias) behind accumulator column c
    if (GATED == 1) wrow = (c < 128) ? (out0 + c) : (a.n_out + out0 + c - 128);
    else wrow = ni * kBN + c;
    const bool in = GATED == 1 ? (out0 + (c & 127) < a.n_out) : (wrow < a.n);
    sb[c] = (bias != nullptr && in) ? to_f32(bias[wrow]) : 0.f;
  }
  __syncwarp();
}

// 2-D bulk-tensor store of one 32-row x 32-column output block (64-byte rows, 64-byte swizzle) from shared
// memory; rows and columns outside the tensor are clipped by the copy engine.
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, const void* src, int c0, int c1) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
               ::"l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(src)), "r"(c0), "r"(c1)
               : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// the issuing thread's earlier bulk stores have finished READING shared memory
__device__ __forceinline__ void bulk_wait_read_all() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
// ... and have completed
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

// One epilogue warp's share of a finished tile: its 32 rows (TMEM lanes at `t_lane`, first row `row0`), half of
// the tile's column steps (`colhalf`). z = acc * alpha + bias, activation, gating, one rounding. Each step
// yields 32 output columns per row; the warp writes them into its 2 KB staging block (row = lane, 16-byte
// chunk c of row r at chunk c ^ ((r >> 1) & 3): the 64-byte swizzle, free of bank conflicts) and one lane hands
// the block to the copy engine. A thread writing its own row straight to global memory costs the L1 one tag
// lookup per row and instruction (32 per store instruction), which made the stores the longest part of the
// epilogue; the bulk store writes whole 64-byte row segments and costs the warp one instruction.
template <int GATED, int ACT, typename OUT, bool FAST = false>
__device__ __forceinline__ void epilogue_columns(const Fc1Args& a, const CUtensorMap* map_y, const float* sb,
                                                 uint8_t* obuf, uint32_t t_lane, int row0, int ni, int colhalf,
                                                 float alpha, int lane) {
  const int out0 = GATED != 0 ? ni * 128 : ni * kBN;  // first output column of the tile
  constexpr int kSteps = GATED != 0 ? 4 : 8;          // steps of 32 output columns per tile
  // FAST (FP8 operands): one special-function instruction per activation; two of them per output are what bounds
  // this epilogue (16 per clock and SM against 128 x 128 outputs per tile), next to an MMA stream twice as fast
  auto actf = [](float g) { return FAST ? act_fwd_fast<ACT>(g) : act_fwd<ACT>(g); };
  // bias values come from shared memory four at a time (all lanes read the same address)
  const float4* sb4 = reinterpret_cast<const float4*>(sb);
#pragma unroll 1
  for (int ch = colhalf * (kSteps / 2); ch < (colhalf + 1) * (kSteps / 2); ++ch) {
    float out[32];
    if constexpr (GATED == 1) {
      float g[32], v[32];
      tc_ld32(t_lane + ch * 32, g);
      tc_ld32(t_lane + 128 + ch * 32, v);
      tc_wait_ld();
#pragma unroll
      for (int j4 = 0; j4 < 8; ++j4) {
        const float4 bg = sb4[ch * 8 + j4], bv = sb4[32 + ch * 8 + j4];
        const float bgs[4] = {bg.x, bg.y, bg.z, bg.w}, bvs[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int j = j4 * 4 + e;
          out[j] = fmaf(v[j], alpha, bvs[e]) * actf(fmaf(g[j], alpha, bgs[e]));
        }
      }
    } else if constexpr (GATED == 2) {
      float z0[32], z1[32];  // accumulator columns (gate, value, gate, ...) of output columns 0..15 and 16..31
      tc_ld32(t_lane + ch * 64, z0);
      tc_ld32(t_lane + ch * 64 + 32, z1);
      tc_wait_ld();
#pragma unroll
      for (int j4 = 0; j4 < 8; ++j4) {
        const float4 b0 = sb4[ch * 16 + j4], b1 = sb4[ch * 16 + 8 + j4];
        out[2 * j4] = fmaf(z0[4 * j4 + 1], alpha, b0.y) * actf(fmaf(z0[4 * j4], alpha, b0.x));
        out[2 * j4 + 1] = fmaf(z0[4 * j4 + 3], alpha, b0.w) * actf(fmaf(z0[4 * j4 + 2], alpha, b0.z));
        out[16 + 2 * j4] = fmaf(z1[4 * j4 + 1], alpha, b1.y) * actf(fmaf(z1[4 * j4], alpha, b1.x));
        out[16 + 2 * j4 + 1] = fmaf(z1[4 * j4 + 3], alpha, b1.w) * actf(fmaf(z1[4 * j4 + 2], alpha, b1.z));
      }
    } else {
      float z[32];
      tc_ld32(t_lane + ch * 32, z);
      tc_wait_ld();
#pragma unroll
      for (int j4 = 0; j4 < 8; ++j4) {
        const float4 b = sb4[ch * 8 + j4];
        out[4 * j4 + 0] = actf(fmaf(z[4 * j4 + 0], alpha, b.x));
        out[4 * j4 + 1] = actf(fmaf(z[4 * j4 + 1], alpha, b.y));
        out[4 * j4 + 2] = actf(fmaf(z[4 * j4 + 2], alpha, b.z));
        out[4 * j4 + 3] = actf(fmaf(z[4 * j4 + 3], alpha, b.w));
      }
    }
    if (lane == 0) bulk_wait_read_all();  // the previous block has left the staging memory
    __syncwarp();
    const int sw = (lane >> 1) & 3;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      uint4 pk;
      pk.x = pack2<OUT>(out[c * 8 + 0], out[c * 8 + 1]);
      pk.y = pack2<OUT>(out[c * 8 + 2], out[c * 8 + 3]);
      pk.z = pack2<OUT>(out[c * 8 + 4], out[c * 8 + 5]);
      pk.w = pack2<OUT>(out[c * 8 + 6], out[c * 8 + 7]);
      *reinterpret_cast<uint4*>(obuf + lane * 64 + ((c ^ sw) << 4)) = pk;
    }
    fence_proxy_async_smem();
    __syncwarp();
    const int col = out0 + ch * 32;
    if (lane == 0 && row0 < a.m && col < a.n_out) {
      tma_store_2d(map_y, obuf, col, row0);
      bulk_commit();
    }
  }
}

// Column sums over the 32 lanes of a warp of 32 values each (lane = row, index = column): five exchange rounds,
// each halving the values a lane holds; lane l ends with the sum of column l, added up in a fixed order.
__device__ __forceinline__ float warp_colsum32(float (&v)[32], int lane) {
#pragma unroll
  for (int half = 16; half >= 1; half >>= 1) {
    const bool upper = (lane & half) != 0;
#pragma unroll
    for (int i = 0; i < half; ++i) {
      const float send = upper ? v[i] : v[i + half];
      const float keep = upper ? v[i + half] : v[i];
      v[i] = keep + __shfl_xor_sync(0xffffffffu, send, half);
    }
  }
  return v[0];
}

// Backward of the gated activation in the epilogue (stacked gating only): the accumulators are the recomputed
// pre-activations z = x W^T + b of the tile, and with the 32 x 32 block of dy fetched by the copy engine into
// the warp's first staging block,
//   dz[:, c]         = dy * value * act'(gate)     (gate half)
//   dz[:, n_out + c] = dy * act(gate)              (value half)
// leave through the other two blocks as two block stores. z itself never reaches memory.
template <int ACT, typename OUT>
__device__ __forceinline__ void epilogue_columns_bwd(const Fc1Args& a, const CUtensorMap* map_dy,
                                                     const CUtensorMap* map_dzg, const CUtensorMap* map_dzv,
                                                     const float* sb, uint8_t* blocks,
                                                     uint64_t* dy_bar, uint32_t& dy_phase, volatile int* abort_flag,
                                                     uint32_t t_lane, int row0, int ni, int colhalf, float alpha, int lane,
                                                     bool& ok) {
  const int out0 = ni * 128;
  const float4* sb4 = reinterpret_cast<const float4*>(sb);
  uint8_t* blk_dy = blocks;
  uint8_t* blk_g = blocks + kOutBlockBytes;
  uint8_t* blk_v = blocks + 2 * kOutBlockBytes;
  const int sw = (lane >> 1) & 3;
#pragma unroll 1
  for (int ch = colhalf * 2; ch < colhalf * 2 + 2; ++ch) {
    const int col = out0 + ch * 32;
    if (lane == 0) {  // rows and columns outside dy are filled with zeros, the byte count is always the full block
      mbar_expect_tx(dy_bar, kOutBlockBytes);
      tma_load_2d(blk_dy, map_dy, dy_bar, col, row0);
    }
    float g[32], v[32];
    tc_ld32(t_lane + ch * 32, g);
    tc_ld32(t_lane + 128 + ch * 32, v);
    tc_wait_ld();
    ok = __all_sync(0xffffffffu, mbar_wait(dy_bar, dy_phase, abort_flag, a.sink, 5));
    if (!ok) return;
    dy_phase ^= 1u;
    float dyv[32];
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const uint4 pk = *reinterpret_cast<const uint4*>(blk_dy + lane * 64 + ((c ^ sw) << 4));
      const uint32_t w4[4] = {pk.x, pk.y, pk.z, pk.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f = unpack_pair<OUT>(w4[e]);
        dyv[c * 8 + 2 * e] = f.x;
        dyv[c * 8 + 2 * e + 1] = f.y;
      }
    }
    float dg[32], dv[32];
#pragma unroll
    for (int j4 = 0; j4 < 8; ++j4) {
      const float4 bg = sb4[ch * 8 + j4], bv = sb4[32 + ch * 8 + j4];
      const float bgs[4] = {bg.x, bg.y, bg.z, bg.w}, bvs[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int j = j4 * 4 + e;
        float grad;
        const float av = act_fwd_grad<ACT>(fmaf(g[j], alpha, bgs[e]), grad);
        dv[j] = dyv[j] * av;
        dg[j] = dyv[j] * fmaf(v[j], alpha, bvs[e]) * grad;
      }
    }
    if (lane == 0) bulk_wait_read_all();  // the previous step's stores have left the two output blocks
    __syncwarp();
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      uint4 pg, pv;
      pg.x = pack2<OUT>(dg[c * 8 + 0], dg[c * 8 + 1]);
      pg.y = pack2<OUT>(dg[c * 8 + 2], dg[c * 8 + 3]);
      pg.z = pack2<OUT>(dg[c * 8 + 4], dg[c * 8 + 5]);
      pg.w = pack2<OUT>(dg[c * 8 + 6], dg[c * 8 + 7]);
      pv.x = pack2<OUT>(dv[c * 8 + 0], dv[c * 8 + 1]);
      pv.y = pack2<OUT>(dv[c * 8 + 2], dv[c * 8 + 3]);
      pv.z = pack2<OUT>(dv[c * 8 + 4], dv[c * 8 + 5]);
      pv.w = pack2<OUT>(dv[c * 8 + 6], dv[c * 8 + 7]);
      *reinterpret_cast<uint4*>(blk_g + lane * 64 + ((c ^ sw) << 4)) = pg;
      *reinterpret_cast<uint4*>(blk_v + lane * 64 + ((c ^ sw) << 4)) = pv;
    }
    fence_proxy_async_smem();
    __syncwarp();  // also: every lane has read its dy before the next step's copy may overwrite the block
    if (lane == 0 && row0 < a.m && col < a.n_out) {
      tma_store_2d(map_dzg, blk_g, col, row0);
      tma_store_2d(map_dzv, blk_v, col, row0);
      bulk_commit();
    }
    if (a.dbias_part != nullptr) {
      // dbias = sum of dz over the tokens, of the values as they are STORED (rounded to the element type, like the
      // reference's dz.sum(0)): this warp's 32 rows give one partial per column, the second stage adds the
      // partials of all row quarters in order. Rows past m and columns past n_out hold zeros (dy is zero there).
#pragma unroll
      for (int j = 0; j < 32; j += 2) {
        const float2 rg = unpack_pair<OUT>(pack2<OUT>(dg[j], dg[j + 1]));
        const float2 rv = unpack_pair<OUT>(pack2<OUT>(dv[j], dv[j + 1]));
        dg[j] = rg.x; dg[j + 1] = rg.y;
        dv[j] = rv.x; dv[j + 1] = rv.y;
      }
      const float sg = warp_colsum32(dg, lane), sv = warp_colsum32(dv, lane);
      if (col + lane < a.n_out && (row0 >> 5) < a.tiles_m * 4) {  // (a pair tile may reach past the last 128-row tile)
        float* row = a.dbias_part + static_cast<size_t>(row0 >> 5) * a.n;
        row[col + lane] = sg;
        row[a.n_out + col + lane] = sv;
      }
    }
  }
}

// ------------------------------------------------------------------ the MMA issuer
// tcgen05.mma with the operand descriptors given as (low word, shared high word): only the 14-bit start
// address in the low word differs between stages and K slices, so the issuing thread keeps one register per
// operand and adds compile-time constants.
template <bool F8, bool PAIR>
__device__ __forceinline__ void tc_mma_split(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t hi, uint32_t idesc,
                                             uint32_t accumulate) {
#define ND_MMA_ASM(GROUP, KIND)                                                                                     \
  asm volatile("{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\tmov.b64 da, {%1, %5};\n\tmov.b64 db, {%2, %5};\n\t"       \
               "setp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::" GROUP ".kind::" KIND " [%0], da, db, %3, p;\n\t}" \
               ::"r"(d_tmem), "r"(a_lo), "r"(b_lo), "r"(idesc), "r"(accumulate), "r"(hi)                             \
               : "memory")
  if constexpr (PAIR) {
    if constexpr (F8) ND_MMA_ASM("2", "f8f6f4");
    else ND_MMA_ASM("2", "f16");
  } else {
    if constexpr (F8) ND_MMA_ASM("1", "f8f6f4");
    else ND_MMA_ASM("1", "f16");
  }
#undef ND_MMA_ASM
}

// "all MMAs issued so far have completed" -> one arrival on `bar`; for a CTA pair, on that barrier in both CTAs
template <bool PAIR> __device__ __forceinline__ void tc_commit_to(uint64_t* bar) {
  if constexpr (PAIR) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(smem_u32(bar)), "h"(static_cast<uint16_t>(3))
                 : "memory");
  } else {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
                 : "memory");
  }
}

// The whole MMA stream of one CTA (or CTA pair), run by ONE thread: `my_tiles` tiles of `k_blocks` stages each.
// The tensor pipe only stays busy if this thread issues one MMA per ~128 cycles while the epilogue warps of the
// same scheduler compete for issue slots, so the loop is kept to the bare chain: the stage ring is unrolled
// (barrier and operand addresses are constants), the operand descriptors are one add away, and the barrier of
// the NEXT stage is polled before the current stage's MMAs are issued so that its answer is there when needed.
template <bool F8, bool PAIR, int STAGES, int STAGE_BYTES>
__device__ __forceinline__ void mma_issue_loop(uint32_t stage0_addr, uint64_t* full, uint64_t* empty,
                                               uint64_t* tmem_full, uint64_t* tmem_empty, uint32_t tmem_base,
                                               uint32_t idesc, int my_tiles, int k_blocks, volatile int* abort_flag,
                                               Fc1Sink sink, int code_tmem, int code_full) {
  const uint32_t a_lo0 = static_cast<uint32_t>(umma_desc(stage0_addr));
  const uint32_t b_lo0 = static_cast<uint32_t>(umma_desc(stage0_addr + kATileBytes));
  const uint32_t hi = static_cast<uint32_t>(umma_desc(stage0_addr) >> 32);
  const long long total_it = static_cast<long long>(my_tiles) * k_blocks;
  int kb = 0, acc = 0;
  uint32_t phase = 0, acc_phase = 0;
  bool ok = true;
  bool ready = total_it > 0 && mbar_try_wait(&full[0], 0);
  for (long long it0 = 0; it0 < total_it && ok; it0 += STAGES) {
#pragma unroll
    for (int st = 0; st < STAGES; ++st) {
      if (it0 + st >= total_it) break;
      if (kb == 0) {  // first stage of a tile: its accumulator must have been drained by the epilogue
        ok = mbar_wait(&tmem_empty[acc], acc_phase ^ 1u, abort_flag, sink, code_tmem);
        if (!ok) break;
      }
      if (!ready) {
        ok = mbar_wait(&full[st], phase, abort_flag, sink, code_full);
        if (!ok) break;
      }
      tc_fence_after();
      const int nst = (st + 1) % STAGES;  // the ring is unrolled: st, nst and `so` below fold to constants
      ready = (it0 + st + 1 < total_it) && mbar_try_wait(&full[nst], st + 1 == STAGES ? phase ^ 1u : phase);
      const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * kBN);
      const uint32_t so = static_cast<uint32_t>(st) * (STAGE_BYTES >> 4);  // descriptor addresses count 16 bytes
      tc_mma_split<F8, PAIR>(d_tmem, a_lo0 + so, b_lo0 + so, hi, idesc, kb != 0 ? 1u : 0u);
#pragma unroll
      for (int kk = 1; kk < kBKBytes / 32; ++kk)  // +32 bytes of K inside the swizzle span = +2 address units
        tc_mma_split<F8, PAIR>(d_tmem, a_lo0 + so + 2u * kk, b_lo0 + so + 2u * kk, hi, idesc, 1u);
      tc_commit_to<PAIR>(&empty[st]);  // the stage is free again once these MMAs have read it
      if (++kb == k_blocks) {
        tc_commit_to<PAIR>(&tmem_full[acc]);  // accumulator complete
        kb = 0;
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1u;
      }
    }
    phase ^= 1u;
  }
}

// ABF: instruction-descriptor operand format (kind::f16: 0 = f16, 1 = bf16; kind::f8f6f4: 0 = e4m3)
// GATED: 0 = y = act(z); 1 = w rows [gate block | value block]; 2 = w rows interleaved (gate0, value0, gate1, ...)
// BWD: the epilogue is the activation backward (map_y / map_y2 describe the gate / value half of dz, each as its
// own [m, n_out] tensor so that the copy engine clips a block at the half's edge; map_dy the incoming gradient)
template <bool F8, int ABF, int GATED, int ACT, typename OUT, bool BWD = false>
__global__ void __launch_bounds__(kThreads, 1)
fc1_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
           const __grid_constant__ CUtensorMap map_y, const __grid_constant__ CUtensorMap map_y2,
           const __grid_constant__ CUtensorMap map_dy, const Fc1Args a) {
  static_assert(!BWD || (GATED == 1 && !F8), "the backward epilogue exists for stacked gating and 16-bit operands");
  constexpr int kS = BWD ? kBwdStages : kStages;
  using Smem = Fc1SmemT<kS, BWD ? 3 : 1>;
  extern __shared__ uint8_t smem_raw[];
  Smem& s = *reinterpret_cast<Smem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  volatile int* abort_flag = &s.abort_flag;
  constexpr int kBKElems = F8 ? 128 : 64;
  const int total_tiles = a.tiles_m * a.tiles_n;

  if (threadIdx.x == 0) {
    for (int i = 0; i < kS; ++i) {
      mbar_init(&s.full[i], 1);
      mbar_init(&s.empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&s.tmem_full[i], 1);
      mbar_init(&s.tmem_empty[i], kEpilogueWarps);
    }
    for (int i = 0; i < kEpilogueWarps; ++i) mbar_init(&s.dy_full[i], 1);
    s.abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_x)) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_w)) : "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&s.tmem_base)),
                 "r"(kTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = s.tmem_base;
  // Programmatic dependent launch: everything above (barriers, tensor memory, tensor-map prefetch) touches no global
  // memory and may run while the previous kernel in the stream drains; nothing below runs before that kernel has
  // completed and its writes are visible. A launch without the attribute passes both instructions at once.
  griddep_launch_dependents();
  griddep_wait();

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer (one thread)
    if (lane == 0) {
      long long w_empty = 0;
      long long* tr0 = a.trace != nullptr ? &w_empty : nullptr;
      const long long t_start = clock64();
      const unsigned long long ns_start = global_ns();
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
        int mi, ni;
        tile_coords(a, t, mi, ni);
        const int m0 = mi * kBM;
        // stacked gating: gate rows [n0, n0+128) and value rows [n_out + n0, ...); otherwise rows [n0, n0+256)
        const int nb0 = GATED == 1 ? ni * 128 : ni * kBN;
        const int nb1 = GATED == 1 ? a.n_out + ni * 128 : ni * kBN + 128;
        for (int kb = 0; kb < a.k_blocks; ++kb) {
          ok = mbar_wait_timed(&s.empty[stage], phase ^ 1u, abort_flag, a.sink, 1, tr0);
          if (!ok) break;
          mbar_expect_tx(&s.full[stage], kStageBytes);
          uint8_t* base = s.stage[stage];
          tma_load_2d(base, &map_x, &s.full[stage], kb * kBKElems, m0);
          tma_load_2d(base + kATileBytes, &map_w, &s.full[stage], kb * kBKElems, nb0);
          tma_load_2d(base + kATileBytes + kBHalfBytes, &map_w, &s.full[stage], kb * kBKElems, nb1);
          if (++stage == kS) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
      if (tr0 != nullptr) {
        atomicAdd(reinterpret_cast<unsigned long long*>(a.trace + 0), static_cast<unsigned long long>(w_empty));
        atomicAdd(reinterpret_cast<unsigned long long*>(a.trace + 5), static_cast<unsigned long long>(clock64() - t_start));
        atomicAdd(reinterpret_cast<unsigned long long*>(a.trace + 7), global_ns() - ns_start);
      }
      if (!ok) {
        // let copies already issued land in shared memory before the CTA may exit
        const unsigned long long t0 = global_ns();
        while (global_ns() - t0 < 200000ull) __nanosleep(1000);
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer (one thread)
    if (lane == 0) {
      const int my_tiles =
          static_cast<int>(blockIdx.x) < total_tiles ? (total_tiles - 1 - static_cast<int>(blockIdx.x)) / static_cast<int>(gridDim.x) + 1 : 0;
      mma_issue_loop<F8, false, kS, kStageBytes>(smem_u32(s.stage[0]), s.full, s.empty, s.tmem_full, s.tmem_empty,
                                                       tmem_base, umma_idesc(ABF), my_tiles, a.k_blocks, abort_flag,
                                                       a.sink, 2, 3);
    }
    __syncwarp();
  } else {
    // ---------------------------------------------------------------- epilogue (8 warps)
    const int q = warp & 3;             // TMEM lane quarter this warp may read
    const int colhalf = (warp - 2) >> 2;   // which half of the tile's column steps this warp takes
    long long w_tfull = 0, busy = 0;
    long long* tr3 = (a.trace != nullptr && lane == 0 && warp == 2) ? &w_tfull : nullptr;
    int acc = 0;
    uint32_t acc_phase = 0;
    [[maybe_unused]] uint32_t dy_phase = 0;
    float alpha = a.alpha_host;
    if (a.alpha_dev != nullptr) alpha *= __ldg(a.alpha_dev) * __ldg(a.alpha_dev + 1);
    bool ok = true;
    for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
      int mi, ni;
      tile_coords(a, t, mi, ni);
      float* sb = s.bias[warp - 2];
      stage_bias<GATED, OUT>(a, sb, ni, lane);
      ok = __all_sync(0xffffffffu, mbar_wait_timed(&s.tmem_full[acc], acc_phase, abort_flag, a.sink, 4, tr3));
      const long long t_busy0 = tr3 != nullptr ? clock64() : 0;
      if (!ok) break;
      tc_fence_after();
      const int row0 = mi * kBM + q * 32;
      const uint32_t t_lane = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + static_cast<uint32_t>(acc * kBN);
      if constexpr (BWD) {
        epilogue_columns_bwd<ACT, OUT>(a, &map_dy, &map_y, &map_y2, sb, s.out[warp - 2][0], &s.dy_full[warp - 2], dy_phase,
                                       abort_flag, t_lane, row0, ni, colhalf, alpha, lane, ok);
        if (!ok) break;
      } else {
        epilogue_columns<GATED, ACT, OUT, F8>(a, &map_y, sb, s.out[warp - 2][0], t_lane, row0, ni, colhalf, alpha, lane);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&s.tmem_empty[acc]);
      if (tr3 != nullptr) busy += clock64() - t_busy0;
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1u;
    }
    if (lane == 0) bulk_wait_all();  // this warp's output blocks are written before the CTA may exit
    if (tr3 != nullptr) {
      atomicAdd(reinterpret_cast<unsigned long long*>(a.trace + 3), static_cast<unsigned long long>(w_tfull));
      atomicAdd(reinterpret_cast<unsigned long long*>(a.trace + 4), static_cast<unsigned long long>(busy));
    }
  }

  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
  }
}

// ------------------------------------------------------------------ two-CTA tiles (cta_group::2)
// A cluster of two CTAs on neighbouring SMs computes a 256 x 256 accumulator tile with one UMMA stream
// issued by the leader (cluster rank 0): each CTA stages the 128 A rows it owns and HALF of the B tile
// (128 weight rows), the tensor cores of both SMs read both halves, and each CTA's tensor memory
// receives the accumulator rows it owns. Per SM that is 32 KB of operands per 128 bytes of K instead
// of 48 KB, which is what the single-CTA kernel runs short of. No multicast loads: every CTA copies
// its own tiles; completion bytes of both CTAs are counted on the leader's mbarrier, and the
// leader's tcgen05.commit signals the "stage free" and "accumulator ready" barriers of both CTAs.
constexpr int kPairStages = 6;
constexpr int kPairStageBytes = kATileBytes + kBHalfBytes;  // 32 KB per CTA and stage

constexpr int kPairBwdStages = 5;  // the backward-dz variant trades one operand stage for two more epilogue blocks

// STAGES operand stages; BLOCKS 32 x 32 staging blocks per epilogue warp (1: output; 3: dy in, two dz halves out)
template <int STAGES, int BLOCKS>
struct __align__(1024) Fc1PairSmemT {
  uint8_t stage[STAGES][kPairStageBytes];
  uint8_t out[kEpilogueWarps][BLOCKS][kOutBlockBytes];
  alignas(16) float bias[kEpilogueWarps][kBN];
  uint64_t full[STAGES];         // used in the leader only: bytes of both CTAs land here
  uint64_t empty[STAGES];        // in each CTA: signalled by the leader's commit
  uint64_t tmem_full[2];         // in each CTA: signalled by the leader's commit
  uint64_t tmem_empty[2];        // used in the leader only: the epilogue warps of both CTAs arrive here
  uint64_t dy_full[kEpilogueWarps];  // backward: the warp's dy block has landed
  uint32_t tmem_base;
  int abort_flag;
};
using Fc1PairSmem = Fc1PairSmemT<kPairStages, 1>;
using Fc1PairBwdSmem = Fc1PairSmemT<kPairBwdStages, 3>;

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t cluster_id_x() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%clusterid.x;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t cluster_count_x() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%nclusterid.x;" : "=r"(r));
  return r;
}
// shared::cluster address of `local` (a shared::cta address) in the CTA of rank `rank`
__device__ __forceinline__ uint32_t mapa_u32(uint32_t local, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// A CTA of a pair that gives up (a bounded wait expired) raises the other CTA's abort flag too, so that the peer's
// roles leave at their next poll instead of running into their own one-second limits one after the other.
__device__ __forceinline__ void abort_peer(volatile int* my_flag, uint32_t peer_flag_cluster_addr) {
  if (*my_flag) asm volatile("st.shared::cluster.b32 [%0], %1;" ::"r"(peer_flag_cluster_addr), "r"(1) : "memory");
}
// 2-D tiled copy into this CTA's shared memory whose completion bytes are counted on an mbarrier that
// may live in the other CTA of the pair (`bar_cluster_addr` is a shared::cluster address).
__device__ __forceinline__ void tma_load_2d_pair(void* dst, const CUtensorMap* map, uint32_t bar_cluster_addr, int c0,
                                                 int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar_cluster_addr), "r"(c0), "r"(c1)
      : "memory");
}
// dense MMA over the CTA pair: M = 256 (128 rows per CTA), N = 256, fp32 accumulator, K-major operands
__host__ __device__ constexpr uint32_t umma_idesc_pair(uint32_t ab_format) {
  return (1u << 4) | (ab_format << 7) | (ab_format << 10) | ((kBN >> 3) << 17) | ((256u >> 4) << 24);
}

// tile t of the pair grid -> (256-row block, n tile); same grouped order as the single-CTA kernel
__device__ __forceinline__ void pair_tile_coords(int tiles_m2, int tiles_n, int t, int& mi, int& ni) {
  const int per_group = kGroupM * tiles_n;
  const int g = t / per_group;
  const int first_m = g * kGroupM;
  const int gm = (tiles_m2 - first_m) < kGroupM ? (tiles_m2 - first_m) : kGroupM;
  const int r = t - g * per_group;
  mi = first_m + r % gm;
  ni = r / gm;
}

// BWD: the epilogue is the activation backward, as in fc1_kernel (map_y / map_y2 the two halves of dz, map_dy the
// incoming gradient)
template <bool F8, int ABF, int GATED, int ACT, typename OUT, bool BWD = false>
__global__ void __launch_bounds__(kThreads, 1)
fc1_pair_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                const __grid_constant__ CUtensorMap map_y, const __grid_constant__ CUtensorMap map_y2,
                const __grid_constant__ CUtensorMap map_dy, const Fc1Args a) {
  static_assert(!BWD || (GATED == 1 && !F8), "the backward epilogue exists for stacked gating and 16-bit operands");
  constexpr int kS = BWD ? kPairBwdStages : kPairStages;
  using Smem = Fc1PairSmemT<kS, BWD ? 3 : 1>;
  extern __shared__ uint8_t smem_raw[];
  Smem& s = *reinterpret_cast<Smem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  volatile int* abort_flag = &s.abort_flag;
  constexpr int kBKElems = F8 ? 128 : 64;
  const uint32_t rank = cluster_ctarank();  // 0 = leader
  const int tiles_m2 = (a.m + 2 * kBM - 1) / (2 * kBM);
  const int total_tiles = tiles_m2 * a.tiles_n;
  const int first_tile = static_cast<int>(cluster_id_x()), tile_step = static_cast<int>(cluster_count_x());

  if (threadIdx.x == 0) {
    for (int i = 0; i < kS; ++i) {
      mbar_init(&s.full[i], 1);
      mbar_init(&s.empty[i], 1);
    }
    for (int i = 0; i < kEpilogueWarps; ++i) mbar_init(&s.dy_full[i], 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&s.tmem_full[i], 1);
      mbar_init(&s.tmem_empty[i], 2 * kEpilogueWarps);
    }
    s.abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_x)) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_w)) : "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&s.tmem_base)),
                 "r"(kTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // the peer's barriers exist before anything is signalled across the pair
  tc_fence_after();
  const uint32_t tmem_base = s.tmem_base;
  const uint32_t peer_abort = mapa_u32(smem_u32(&s.abort_flag), rank ^ 1u);
  // Programmatic dependent launch: everything above (barriers, tensor memory, tensor-map prefetch) touches no global
  // memory and may run while the previous kernel in the stream drains; nothing below runs before that kernel has
  // completed and its writes are visible. A launch without the attribute passes both instructions at once.
  griddep_launch_dependents();
  griddep_wait();

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer (one thread in each CTA)
    if (lane == 0) {
      const long long t_start = clock64();
      const unsigned long long ns_start = global_ns();
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = first_tile; t < total_tiles && ok; t += tile_step) {
        int mi, ni;
        pair_tile_coords(tiles_m2, a.tiles_n, t, mi, ni);
        const int m0 = mi * 2 * kBM + static_cast<int>(rank) * kBM;  // this CTA's 128 rows of the 256-row tile
        // this CTA's half of the B tile: stacked gating -> leader takes the gate rows, peer the value rows
        const int nb =
            GATED == 1 ? (rank == 0 ? ni * 128 : a.n_out + ni * 128) : ni * kBN + static_cast<int>(rank) * 128;
        for (int kb = 0; kb < a.k_blocks; ++kb) {
          ok = mbar_wait(&s.empty[stage], phase ^ 1u, abort_flag, a.sink, 11);
          if (!ok) break;
          if (rank == 0) mbar_expect_tx(&s.full[stage], 2 * kPairStageBytes);  // both CTAs' bytes
          const uint32_t leader_full = mapa_u32(smem_u32(&s.full[stage]), 0);
          uint8_t* base = s.stage[stage];
          tma_load_2d_pair(base, &map_x, leader_full, kb * kBKElems, m0);
          tma_load_2d_pair(base + kATileBytes, &map_w, leader_full, kb * kBKElems, nb);
          if (++stage == kS) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
      if (a.trace != nullptr) {
        atomicAdd(reinterpret_cast<unsigned long long*>(a.trace + 5), static_cast<unsigned long long>(clock64() - t_start));
        atomicAdd(reinterpret_cast<unsigned long long*>(a.trace + 7), global_ns() - ns_start);
      }
      abort_peer(abort_flag, peer_abort);
      if (!ok) {
        const unsigned long long t0 = global_ns();
        while (global_ns() - t0 < 200000ull) __nanosleep(1000);
      }
    }
    __syncwarp();
  } else if (warp == 1 && rank == 0) {
    // ---------------------------------------------------------------- MMA issuer (one thread of the leader)
    if (lane == 0) {
      const int my_tiles = first_tile < total_tiles ? (total_tiles - 1 - first_tile) / tile_step + 1 : 0;
      mma_issue_loop<F8, true, kS, kPairStageBytes>(smem_u32(s.stage[0]), s.full, s.empty, s.tmem_full,
                                                              s.tmem_empty, tmem_base, umma_idesc_pair(ABF), my_tiles,
                                                              a.k_blocks, abort_flag, a.sink, 12, 13);
      abort_peer(abort_flag, peer_abort);
    }
    __syncwarp();
  } else if (warp >= 2) {
    // ---------------------------------------------------------------- epilogue (8 warps, both CTAs)
    const int q = warp & 3;
    const int colhalf = (warp - 2) >> 2;
    int acc = 0;
    uint32_t acc_phase = 0;
    [[maybe_unused]] uint32_t dy_phase = 0;
    float alpha = a.alpha_host;
    if (a.alpha_dev != nullptr) alpha *= __ldg(a.alpha_dev) * __ldg(a.alpha_dev + 1);
    bool ok = true;
    for (int t = first_tile; t < total_tiles && ok; t += tile_step) {
      int mi, ni;
      pair_tile_coords(tiles_m2, a.tiles_n, t, mi, ni);
      float* sb = s.bias[warp - 2];
      stage_bias<GATED, OUT>(a, sb, ni, lane);
      ok = __all_sync(0xffffffffu, mbar_wait(&s.tmem_full[acc], acc_phase, abort_flag, a.sink, 14));
      if (!ok) break;
      tc_fence_after();
      const int row0 = mi * 2 * kBM + static_cast<int>(rank) * kBM + q * 32;
      const uint32_t t_lane = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + static_cast<uint32_t>(acc * kBN);
      if constexpr (BWD) {
        epilogue_columns_bwd<ACT, OUT>(a, &map_dy, &map_y, &map_y2, sb, s.out[warp - 2][0], &s.dy_full[warp - 2], dy_phase,
                                       abort_flag, t_lane, row0, ni, colhalf, alpha, lane, ok);
        if (!ok) break;
      } else {
        epilogue_columns<GATED, ACT, OUT, F8>(a, &map_y, sb, s.out[warp - 2][0], t_lane, row0, ni, colhalf, alpha, lane);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(mapa_u32(smem_u32(&s.tmem_empty[acc]), 0));  // the leader counts both CTAs
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1u;
    }
    if (lane == 0) {
      abort_peer(abort_flag, peer_abort);
      bulk_wait_all();
    }
  }

  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // neither CTA frees tensor memory or exits while the other may still signal it
  tc_fence_after();
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
  }
}

// ------------------------------------------------------------------ host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  // cuTensorMapEncodeTiled is a driver call and wants a CUDA context current on the calling thread. A thread that
  // has only used cached runtime state so far (PyTorch's autograd worker calling a backward entry point first) may
  // have none bound yet: one runtime call that needs the context binds the device's primary context to the thread.
  static thread_local bool context_bound = false;
  if (!context_bound) {
    (void)cudaFree(nullptr);
    context_bound = true;
  }
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
    else
      (void)cudaGetLastError();
  });
  return fn;
}

// rows x k matrix, k contiguous; box = 128 bytes of k x 128 rows, 128B swizzle, zero fill out of bounds
static bool make_map(CUtensorMap* map, CUtensorMapDataType dt, int elem_bytes, const void* base, long long rows,
                     long long k) {
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) return false;
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(k), static_cast<cuuint64_t>(rows)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(k) * elem_bytes};
  const cuuint32_t box[2] = {static_cast<cuuint32_t>(kBKBytes / elem_bytes), 128u};
  const cuuint32_t estr[2] = {1u, 1u};
  return fn(map, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <bool F8, int ABF, typename OUT>
static const void* pick_fc1(int act, int gated) {
  const bool silu = act == ND_ACT_SILU;
  switch (gated) {
    case 1:
      return silu ? (const void*)fc1_kernel<F8, ABF, 1, ND_ACT_SILU, OUT> : (const void*)fc1_kernel<F8, ABF, 1, ND_ACT_GELU, OUT>;
    case 2:
      return silu ? (const void*)fc1_kernel<F8, ABF, 2, ND_ACT_SILU, OUT> : (const void*)fc1_kernel<F8, ABF, 2, ND_ACT_GELU, OUT>;
    default:
      if (act == ND_ACT_NONE) return (const void*)fc1_kernel<F8, ABF, 0, ND_ACT_NONE, OUT>;
      return silu ? (const void*)fc1_kernel<F8, ABF, 0, ND_ACT_SILU, OUT> : (const void*)fc1_kernel<F8, ABF, 0, ND_ACT_GELU, OUT>;
  }
}

template <bool F8, int ABF, typename OUT>
static const void* pick_fc1_pair(int act, int gated) {
  const bool silu = act == ND_ACT_SILU;
  switch (gated) {
    case 1:
      return silu ? (const void*)fc1_pair_kernel<F8, ABF, 1, ND_ACT_SILU, OUT> : (const void*)fc1_pair_kernel<F8, ABF, 1, ND_ACT_GELU, OUT>;
    case 2:
      return silu ? (const void*)fc1_pair_kernel<F8, ABF, 2, ND_ACT_SILU, OUT> : (const void*)fc1_pair_kernel<F8, ABF, 2, ND_ACT_GELU, OUT>;
    default:
      if (act == ND_ACT_NONE) return (const void*)fc1_pair_kernel<F8, ABF, 0, ND_ACT_NONE, OUT>;
      return silu ? (const void*)fc1_pair_kernel<F8, ABF, 0, ND_ACT_SILU, OUT> : (const void*)fc1_pair_kernel<F8, ABF, 0, ND_ACT_GELU, OUT>;
  }
}

static std::atomic<int> g_fc1_pdl{1};    // 1 = launch with programmatic stream serialization
static std::atomic<int> g_fc1_pair{-1};  // -1 = choose per problem
static std::atomic<long long*> g_fc1_trace{nullptr};


// ------------------------------------------------------------------ the two GEMMs of the FC1 backward
// dx = dz W   (dz [M, 2I], W [2I, H]: the reduction runs over 2I, W's rows)         A K-major,  B MN-major
// dW = dz^T x (dz [M, 2I], x [M, H]:  the reduction runs over the M token rows)      A MN-major, B MN-major
// In both the B operand - and for dW the A operand too - is contiguous along its M/N dimension, not along K. UMMA
// takes such operands in place ("MN-major", instruction-descriptor bits 15 / 16), so nothing is transposed or
// copied. An MN-major tile is staged as boxes of 64 elements (128 bytes, along M/N) x 64 K-rows with the 128-byte
// swizzle: K-row r of a box sits at r * 128 bytes, 8-row groups are 1024 bytes apart (the descriptor's stride
// offset), boxes 8192 bytes apart (its leading offset), and one UMMA of K = 16 consumes two 8-row groups, so the
// k-th slice of a stage starts 2048 k bytes into it.
// Tiles are 128 x 192: H = 1152 is six of them exactly (a 256-wide tile wastes 10 % there), 192 fp32 columns
// twice fit tensor memory, and a CTA reads 10 KB of operands per MMA of 96 cycles, within what shared memory
// delivers. One CTA per SM, persistent over tiles; warp 0 copies, warp 1 issues, warps 2-5 drain one 32-row
// quarter of the accumulator each (no bias, no activation: the epilogue is a rounding).
constexpr int kGemmBN = 192;
constexpr int kGemmStages = 5;
constexpr int kGemmBoxBytes = 64 * 128;                       // one MN-major box: 64 K-rows of 128 bytes
constexpr int kGemmBBytes = (kGemmBN / 64) * kGemmBoxBytes;   // 24 KB
constexpr int kGemmStageBytes = kATileBytes + kGemmBBytes;    // 40 KB
constexpr int kGemmThreads = 64 + 4 * 32;

struct __align__(1024) GemmSmem {
  uint8_t stage[kGemmStages][kGemmStageBytes];
  uint8_t out[4][kOutBlockBytes];
  uint64_t full[kGemmStages];
  uint64_t empty[kGemmStages];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint32_t tmem_base;
  int abort_flag;
};

struct GemmArgs {
  Fc1Sink sink;
  int m, n, k;
  int tiles_m, tiles_n, k_blocks;
};

// MN-major, 128B-swizzled operand tile (see above): leading offset 8192 bytes, stride offset 1024 bytes
__device__ __forceinline__ uint64_t umma_desc_mn(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);
  d |= static_cast<uint64_t>(kGemmBoxBytes >> 4) << 16;
  d |= static_cast<uint64_t>(1024 >> 4) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(2) << 61;
  return d;
}

__host__ __device__ constexpr uint32_t umma_idesc_gemm(uint32_t ab_format, bool a_mn) {
  return (1u << 4) | (ab_format << 7) | (ab_format << 10) | (a_mn ? (1u << 15) : 0u) | (1u << 16) |
         ((kGemmBN >> 3) << 17) | ((kBM >> 4) << 24);
}

template <int ABF, bool A_MN, typename OUT>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_bwd_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                const __grid_constant__ CUtensorMap map_c, const GemmArgs a) {
  extern __shared__ uint8_t smem_raw[];
  GemmSmem& s = *reinterpret_cast<GemmSmem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  volatile int* abort_flag = &s.abort_flag;
  const int total_tiles = a.tiles_m * a.tiles_n;
  auto coords = [&](int t, int& mi, int& ni) {  // groups of 8 row tiles share their B tiles in L2
    const int per_group = kGroupM * a.tiles_n;
    const int g = t / per_group, first_m = g * kGroupM;
    const int gm = (a.tiles_m - first_m) < kGroupM ? (a.tiles_m - first_m) : kGroupM;
    const int r = t - g * per_group;
    mi = first_m + r % gm;
    ni = r / gm;
  };

  if (threadIdx.x == 0) {
    for (int i = 0; i < kGemmStages; ++i) {
      mbar_init(&s.full[i], 1);
      mbar_init(&s.empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&s.tmem_full[i], 1);
      mbar_init(&s.tmem_empty[i], 4);
    }
    s.abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_a)) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_b)) : "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&s.tmem_base)),
                 "r"(kTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = s.tmem_base;
  // Programmatic dependent launch: everything above (barriers, tensor memory, tensor-map prefetch) touches no global
  // memory and may run while the previous kernel in the stream drains; nothing below runs before that kernel has
  // completed and its writes are visible. A launch without the attribute passes both instructions at once.
  griddep_launch_dependents();
  griddep_wait();

  if (warp == 0) {
    if (lane == 0) {  // ---------------------------------------------------------- copies
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
        int mi, ni;
        coords(t, mi, ni);
        const int m0 = mi * kBM, n0 = ni * kGemmBN;
        for (int kb = 0; kb < a.k_blocks; ++kb) {
          ok = mbar_wait(&s.empty[stage], phase ^ 1u, abort_flag, a.sink, 21);
          if (!ok) break;
          mbar_expect_tx(&s.full[stage], kGemmStageBytes);
          uint8_t* base = s.stage[stage];
          if constexpr (A_MN) {
            tma_load_2d(base, &map_a, &s.full[stage], m0, kb * 64);
            tma_load_2d(base + kGemmBoxBytes, &map_a, &s.full[stage], m0 + 64, kb * 64);
          } else {
            tma_load_2d(base, &map_a, &s.full[stage], kb * 64, m0);
          }
#pragma unroll
          for (int j = 0; j < kGemmBN / 64; ++j)
            tma_load_2d(base + kATileBytes + j * kGemmBoxBytes, &map_b, &s.full[stage], n0 + 64 * j, kb * 64);
          if (++stage == kGemmStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
      if (!ok) {  // let copies already issued land in shared memory before the CTA may exit
        const unsigned long long t0 = global_ns();
        while (global_ns() - t0 < 200000ull) __nanosleep(1000);
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (lane == 0) {  // ---------------------------------------------------------- MMA issue
      const int my_tiles = static_cast<int>(blockIdx.x) < total_tiles
                               ? (total_tiles - 1 - static_cast<int>(blockIdx.x)) / static_cast<int>(gridDim.x) + 1 : 0;
      constexpr uint32_t idesc = umma_idesc_gemm(ABF, A_MN);
      const uint32_t stage0 = smem_u32(s.stage[0]);
      const uint64_t a_d0 = A_MN ? umma_desc_mn(stage0) : umma_desc(stage0);
      const uint64_t b_d0 = umma_desc_mn(stage0 + kATileBytes);
      const uint32_t a_hi = static_cast<uint32_t>(a_d0 >> 32), b_hi = static_cast<uint32_t>(b_d0 >> 32);
      const uint32_t a_lo0 = static_cast<uint32_t>(a_d0), b_lo0 = static_cast<uint32_t>(b_d0);
      constexpr uint32_t a_step = A_MN ? (2048u >> 4) : 2u;  // one K = 16 slice further, in 16-byte address units
      int stage = 0, acc = 0;
      uint32_t phase = 0, acc_phase = 0;
      bool ok = true;
      for (int i = 0; i < my_tiles && ok; ++i) {
        ok = mbar_wait(&s.tmem_empty[acc], acc_phase ^ 1u, abort_flag, a.sink, 22);
        if (!ok) break;
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * 256);
        for (int kb = 0; kb < a.k_blocks; ++kb) {
          ok = mbar_wait(&s.full[stage], phase, abort_flag, a.sink, 23);
          if (!ok) break;
          tc_fence_after();
          const uint32_t so = static_cast<uint32_t>(stage) * (kGemmStageBytes >> 4);
#pragma unroll
          for (int kk = 0; kk < 4; ++kk) {
            const uint32_t al = a_lo0 + so + a_step * kk, bl = b_lo0 + so + (2048u >> 4) * kk;
            const uint32_t accum = (kb != 0 || kk != 0) ? 1u : 0u;
            asm volatile("{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\tmov.b64 da, {%1, %5};\n\tmov.b64 db, {%2, %6};\n\t"
                         "setp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %3, p;\n\t}"
                         ::"r"(d_tmem), "r"(al), "r"(bl), "r"(idesc), "r"(accum), "r"(a_hi), "r"(b_hi)
                         : "memory");
          }
          tc_commit_to<false>(&s.empty[stage]);
          if (++stage == kGemmStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (!ok) break;
        tc_commit_to<false>(&s.tmem_full[acc]);
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1u;
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------------------ epilogue: 4 warps, 32 rows each
    const int q = warp & 3;
    uint8_t* obuf = s.out[warp - 2];
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
      int mi, ni;
      coords(t, mi, ni);
      ok = __all_sync(0xffffffffu, mbar_wait(&s.tmem_full[acc], acc_phase, abort_flag, a.sink, 24));
      if (!ok) break;
      tc_fence_after();
      const int row0 = mi * kBM + q * 32;
      const uint32_t t_lane = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + static_cast<uint32_t>(acc * 256);
#pragma unroll 1
      for (int ch = 0; ch < kGemmBN / 32; ++ch) {
        float z[32];
        tc_ld32(t_lane + ch * 32, z);
        tc_wait_ld();
        if (lane == 0) bulk_wait_read_all();  // the previous block has left the staging memory
        __syncwarp();
        const int sw = (lane >> 1) & 3;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint4 pk;
          pk.x = pack2<OUT>(z[c * 8 + 0], z[c * 8 + 1]);
          pk.y = pack2<OUT>(z[c * 8 + 2], z[c * 8 + 3]);
          pk.z = pack2<OUT>(z[c * 8 + 4], z[c * 8 + 5]);
          pk.w = pack2<OUT>(z[c * 8 + 6], z[c * 8 + 7]);
          *reinterpret_cast<uint4*>(obuf + lane * 64 + ((c ^ sw) << 4)) = pk;
        }
        fence_proxy_async_smem();
        __syncwarp();
        const int col = ni * kGemmBN + ch * 32;
        if (lane == 0 && row0 < a.m && col < a.n) {
          tma_store_2d(&map_c, obuf, col, row0);
          bulk_commit();
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&s.tmem_empty[acc]);
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1u;
    }
    if (lane == 0) bulk_wait_all();
  }

  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
  }
}

// ------------------------------------------------------------------ the same GEMMs over CTA pairs, K split evenly
// What the tensor pipe charges for an MMA here does not depend on N: measured with a free-running issue loop, an
// MMA of K = 16 takes ~160 cycles on a single CTA (M = 128) and ~128 cycles on a CTA pair (M = 256, 128 rows per
// CTA), whether N is 128, 192 or 256 - the rows stream through, the columns lie side by side. So the cost of a GEMM
// is its NUMBER of MMAs, a 128 x 192 tile uses 60 % of the pipe at best, and the efficient shape is the pair's
// 256 x 256 tile. H = 1152 is four and a half of those: a row block costs five tiles' worth of MMAs (the half tile
// is charged like a full one), and 160 or 180 tiles of 144 or 128 k-blocks do not divide over 74 clusters. Hence
// the k-blocks of all tiles are laid end to end and cut into one contiguous range per cluster, equal to within one
// k-block ("stream-K"). A range is at least one tile long, so a tile is cut at most once: the two clusters that
// share it each write their fp32 partial accumulator to the caller's workspace and count themselves in, per warp
// quarter; whoever comes second adds the two (a sum of two is the same in either order, so the result does not
// depend on who that is) and writes the tile. Nobody waits for anybody.
// Each CTA stages ITS 128 rows of A and ITS half of the tile's B columns, the leader's one thread issues the MMAs
// over both CTAs' shared memory, and each CTA drains its own 128 lanes of tensor memory.
constexpr int kGpStages = 6;
constexpr int kGpBHalfBytes = 2 * kGemmBoxBytes;             // a CTA's half of a 256-wide B tile: two boxes, 16 KB
constexpr int kGpStageBytes = kATileBytes + kGpBHalfBytes;   // 32 KB
constexpr int kGpCounterBytes = 4096;                        // head of the workspace: arrival counters
constexpr size_t kGpPartialFloats = 128 * 256;               // one CTA's share of a partial tile

struct __align__(1024) GemmPairSmem {
  uint8_t stage[kGpStages][kGpStageBytes];
  uint8_t out[4][kOutBlockBytes];
  uint64_t full[kGpStages];    // used in the leader only: counts the bytes of both CTAs
  uint64_t empty[kGpStages];   // in each CTA: signalled by the leader's commits (multicast to the pair)
  uint64_t tmem_full[2];       // in each CTA, likewise
  uint64_t tmem_empty[2];      // used in the leader only: the epilogue warps of both CTAs arrive here
  uint32_t tmem_base;
  int abort_flag;
};

struct GemmPairArgs {
  Fc1Sink sink;
  long long* trace;   // nullable: cycle counters of the leader's issuing thread (see nd_tune_fc1_trace)
  int* counters;      // zeroed before the launch; [boundary][rank][quarter]
  float* partials;    // [boundary][side][rank][quarter][chunk][float4 index][lane][4]
  long long total_it; // tiles x k-blocks
  int m, n, k;
  int tiles_n, k_blocks;
};

// The segments (tile, k-block range) of one cluster's share, in the order every role of both CTAs walks them: the
// cut tile at the END of the range first, then the cut tile at its beginning, then the whole tiles in between. Both
// halves of a shared tile are then computed early by their two clusters, and the second one's finishing pass over
// the partials runs under the MMAs of the tiles that follow instead of at the end of the kernel.
struct SegWalk {
  long long g0, g1, g;   // the range, and the next whole-tile position
  int kbs, tiles_n, step;
  __device__ __forceinline__ SegWalk(const GemmPairArgs& a, int cluster, int clusters)
      : kbs(a.k_blocks), tiles_n(a.tiles_n), step(0) {
    const long long base = a.total_it / clusters, rem = a.total_it % clusters;
    g0 = cluster * base + (cluster < rem ? cluster : rem);
    g1 = g0 + base + (cluster < rem ? 1 : 0);
    g = g0;
  }
  __device__ __forceinline__ long long length() const { return g1 - g0; }
  __device__ __forceinline__ void tile_of(long long t, int& row_block, int& col_tile) const {
    row_block = static_cast<int>(t / tiles_n);
    col_tile = static_cast<int>(t - static_cast<long long>(row_block) * tiles_n);
  }
  // the tile cut by the end of the range (continued by the next cluster); `take` removes it from the range
  __device__ __forceinline__ int tail_len() const {
    const long long t = g1 / kbs;
    const int tail = static_cast<int>(g1 - t * kbs);
    return (tail != 0 && t * kbs >= g0) ? tail : 0;  // (a range inside one tile cannot occur: a range is >= a tile)
  }
  // the tile cut by the beginning of the range (begun by the previous cluster)
  __device__ __forceinline__ int head_len() const {
    const long long t = g0 / kbs;
    const int off = static_cast<int>(g0 - t * kbs);
    return off != 0 ? kbs - off : 0;
  }
  __device__ __forceinline__ bool next(int& row_block, int& col_tile, int& kb0, int& kb1) {
    // steps 0 and 1: the two cut tiles, the SHORTER one first - its epilogue (store the partial, maybe finish the
    // tile) then runs under the longer one's MMAs and has freed its accumulator when the first whole tile wants it
    while (step < 2) {
      const int tail = tail_len(), head = head_len();
      const bool tail_turn = (step == 0) == (tail <= head);
      ++step;
      if (tail_turn && tail != 0) {
        tile_of(g1 / kbs, row_block, col_tile);
        kb0 = 0;
        kb1 = tail;
        return true;
      }
      if (!tail_turn && head != 0) {
        tile_of(g0 / kbs, row_block, col_tile);
        kb0 = kbs - head;
        kb1 = kbs;
        return true;
      }
    }
    if (step == 2) {  // the whole tiles in between
      step = 3;
      g = g0 + head_len();
      g1 -= tail_len();
    }
    if (g >= g1) return false;
    tile_of(g / kbs, row_block, col_tile);
    kb0 = 0;
    kb1 = kbs;
    g += kbs;
    return true;
  }
};

__host__ __device__ constexpr uint32_t umma_idesc_gemm_pair(uint32_t ab_format, bool a_mn, uint32_t n) {
  return (1u << 4) | (ab_format << 7) | (ab_format << 10) | (a_mn ? (1u << 15) : 0u) | (1u << 16) | ((n >> 3) << 17) |
         ((256u >> 4) << 24);
}

template <int ABF, bool A_MN, typename OUT>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_bwd_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                     const __grid_constant__ CUtensorMap map_c, const GemmPairArgs a) {
  extern __shared__ uint8_t smem_raw[];
  GemmPairSmem& s = *reinterpret_cast<GemmPairSmem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  volatile int* abort_flag = &s.abort_flag;
  const uint32_t rank = cluster_ctarank();  // 0 = leader
  const int cluster = static_cast<int>(cluster_id_x()), clusters = static_cast<int>(cluster_count_x());

  if (threadIdx.x == 0) {
    for (int i = 0; i < kGpStages; ++i) {
      mbar_init(&s.full[i], 1);
      mbar_init(&s.empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&s.tmem_full[i], 1);
      mbar_init(&s.tmem_empty[i], 2 * 4);
    }
    s.abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_a)) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_b)) : "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&s.tmem_base)),
                 "r"(kTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // the peer's barriers exist before anything is signalled across the pair
  tc_fence_after();
  const uint32_t tmem_base = s.tmem_base;
  const uint32_t peer_abort = mapa_u32(smem_u32(&s.abort_flag), rank ^ 1u);
  // Programmatic dependent launch: everything above (barriers, tensor memory, tensor-map prefetch) touches no global
  // memory and may run while the previous kernel in the stream drains; nothing below runs before that kernel has
  // completed and its writes are visible. A launch without the attribute passes both instructions at once.
  griddep_launch_dependents();
  griddep_wait();

  if (warp == 0) {
    if (lane == 0) {  // ---------------------------------------------------------- copies (one thread in each CTA)
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      SegWalk walk(a, cluster, clusters);
      int rb, ct, kb0, kb1;
      while (ok && walk.next(rb, ct, kb0, kb1)) {
        const int wide = (a.n - ct * 256) > 128 ? 1 : 0;                  // the last column tile may be a half tile
        const int m0 = rb * 2 * kBM + static_cast<int>(rank) * kBM;       // this CTA's 128 rows of the tile
        const int n0 = ct * 256 + static_cast<int>(rank) * (wide ? 128 : 64);  // this CTA's half of the columns
        const uint32_t both = 2u * static_cast<uint32_t>(kATileBytes + (wide ? 2 : 1) * kGemmBoxBytes);
        for (int kb = kb0; kb < kb1; ++kb) {
          ok = mbar_wait(&s.empty[stage], phase ^ 1u, abort_flag, a.sink, 31);
          if (!ok) break;
          if (rank == 0) mbar_expect_tx(&s.full[stage], both);
          const uint32_t leader_full = mapa_u32(smem_u32(&s.full[stage]), 0);
          uint8_t* base = s.stage[stage];
          if constexpr (A_MN) {
            tma_load_2d_pair(base, &map_a, leader_full, m0, kb * 64);
            tma_load_2d_pair(base + kGemmBoxBytes, &map_a, leader_full, m0 + 64, kb * 64);
          } else {
            tma_load_2d_pair(base, &map_a, leader_full, kb * 64, m0);
          }
          tma_load_2d_pair(base + kATileBytes, &map_b, leader_full, n0, kb * 64);
          if (wide) tma_load_2d_pair(base + kATileBytes + kGemmBoxBytes, &map_b, leader_full, n0 + 64, kb * 64);
          if (++stage == kGpStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
      abort_peer(abort_flag, peer_abort);
      if (!ok) {  // let copies already issued land in shared memory before the CTA may exit
        const unsigned long long t0 = global_ns();
        while (global_ns() - t0 < 200000ull) __nanosleep(1000);
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (lane == 0 && rank == 0) {  // ---------------------------------------------- MMA issue (the leader's thread)
      // The tensor pipe takes only a shallow queue of MMAs: the barrier of the NEXT stage is polled before the
      // current stage's MMAs are issued, and the stage ring is unrolled so that addresses fold to constants.
      const long long t_start = a.trace != nullptr ? clock64() : 0;
      const uint32_t stage0 = smem_u32(s.stage[0]);
      const uint64_t a_d0 = A_MN ? umma_desc_mn(stage0) : umma_desc(stage0);
      const uint64_t b_d0 = umma_desc_mn(stage0 + kATileBytes);
      const uint32_t a_hi = static_cast<uint32_t>(a_d0 >> 32), b_hi = static_cast<uint32_t>(b_d0 >> 32);
      const uint32_t a_lo0 = static_cast<uint32_t>(a_d0), b_lo0 = static_cast<uint32_t>(b_d0);
      constexpr uint32_t a_step = A_MN ? (2048u >> 4) : 2u;  // one K = 16 slice further, in 16-byte address units
      constexpr uint32_t b_step = 2048u >> 4;
      long long waited_full = 0, waited_acc = 0;
      long long* trf = a.trace != nullptr ? &waited_full : nullptr;
      long long* tra = a.trace != nullptr ? &waited_acc : nullptr;
      SegWalk walk(a, cluster, clusters);
      const long long total_it = walk.length();
      int rb, ct, kb = 0, kb0 = 0, kb1 = 0, acc = 0;
      uint32_t phase = 0, acc_phase = 0, idesc = 0, d_tmem = 0;
      bool ok = true;
      bool ready = total_it > 0 && mbar_try_wait(&s.full[0], 0);
      for (long long it0 = 0; it0 < total_it && ok; it0 += kGpStages) {
#pragma unroll
        for (int st = 0; st < kGpStages; ++st) {
          if (it0 + st >= total_it) break;
          if (kb == kb1) {  // a new segment: its accumulator must have been drained by the epilogues
            walk.next(rb, ct, kb0, kb1);
            kb = kb0;
            idesc = umma_idesc_gemm_pair(ABF, A_MN, (a.n - ct * 256) > 128 ? 256u : 128u);
            d_tmem = tmem_base + static_cast<uint32_t>(acc * 256);
            ok = mbar_wait_timed(&s.tmem_empty[acc], acc_phase ^ 1u, abort_flag, a.sink, 32, tra);
            if (!ok) break;
          }
          if (!ready) {
            ok = mbar_wait_timed(&s.full[st], phase, abort_flag, a.sink, 33, trf);
            if (!ok) break;
          }
          tc_fence_after();
          const int nst = (st + 1) % kGpStages;  // the ring is unrolled: st and nst fold to constants
          ready = (it0 + st + 1 < total_it) && mbar_try_wait(&s.full[nst], st + 1 == kGpStages ? phase ^ 1u : phase);
          const uint32_t so = static_cast<uint32_t>(st) * (kGpStageBytes >> 4);
#pragma unroll
          for (int kk = 0; kk < 4; ++kk) {
            const uint32_t al = a_lo0 + so + a_step * kk, bl = b_lo0 + so + b_step * kk;
            const uint32_t accum = (kb != kb0 || kk != 0) ? 1u : 0u;
            asm volatile("{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\tmov.b64 da, {%1, %5};\n\tmov.b64 db, {%2, %6};\n\t"
                         "setp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::2.kind::f16 [%0], da, db, %3, p;\n\t}"
                         ::"r"(d_tmem), "r"(al), "r"(bl), "r"(idesc), "r"(accum), "r"(a_hi), "r"(b_hi)
                         : "memory");
          }
          tc_commit_to<true>(&s.empty[st]);  // frees the stage in both CTAs
          if (++kb == kb1) {
            tc_commit_to<true>(&s.tmem_full[acc]);  // the segment's accumulator is complete: both CTAs' epilogues
            acc ^= 1;
            if (acc == 0) acc_phase ^= 1u;
          }
        }
        phase ^= 1u;
      }
      abort_peer(abort_flag, peer_abort);
      if (a.trace != nullptr) {
        atomicAdd(reinterpret_cast<unsigned long long*>(a.trace + 5), static_cast<unsigned long long>(clock64() - t_start));
        atomicAdd(reinterpret_cast<unsigned long long*>(a.trace + 6), 1ull);
        atomicAdd(reinterpret_cast<unsigned long long*>(a.trace + 7), static_cast<unsigned long long>(total_it));
        atomicAdd(reinterpret_cast<unsigned long long*>(a.trace + 0), static_cast<unsigned long long>(waited_acc));
        atomicAdd(reinterpret_cast<unsigned long long*>(a.trace + 1), static_cast<unsigned long long>(waited_full));
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------------------ epilogue: 4 warps, 32 rows each
    const int q = warp & 3;
    uint8_t* obuf = s.out[warp - 2];
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    SegWalk walk(a, cluster, clusters);
    int rb, ct, kb0, kb1;
    while (ok && walk.next(rb, ct, kb0, kb1)) {
      ok = __all_sync(0xffffffffu, mbar_wait(&s.tmem_full[acc], acc_phase, abort_flag, a.sink, 34));
      if (!ok) break;
      tc_fence_after();
      const int row0 = rb * 2 * kBM + static_cast<int>(rank) * kBM + q * 32;
      const int col0 = ct * 256;
      const uint32_t t_lane = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + static_cast<uint32_t>(acc * 256);
      const int chunks = (a.n - col0) > 128 ? 8 : 4;
      const bool whole = kb0 == 0 && kb1 == a.k_blocks;
      const float* other = nullptr;
      bool write_out = whole;
      if (!whole) {
        // this tile is shared with the neighbouring cluster: side 1 continues what cluster - 1 began, side 0 begins
        // what cluster + 1 continues. Store the partial, count in; the second of the two to arrive finishes the tile.
        const int side = kb0 > 0 ? 1 : 0;
        const size_t boundary = static_cast<size_t>(side ? cluster - 1 : cluster);
        // a warp's share of a partial is private to the two warps (same rank, same quarter) that exchange it, so it
        // is laid out for them: [chunk][float4 index][lane] - every store and load instruction moves 512 contiguous
        // bytes (rows a kilobyte apart, one float4 per lane, took ten times as long)
        float* mine = a.partials + ((((boundary * 2 + side) * 2 + rank) * 4 + q) * 8) * 1024 + lane * 4;
        other = a.partials + ((((boundary * 2 + (side ^ 1)) * 2 + rank) * 4 + q) * 8) * 1024 + lane * 4;
#pragma unroll 1
        for (int ch = 0; ch < chunks; ++ch) {
          float z[32];
          tc_ld32(t_lane + ch * 32, z);
          tc_wait_ld();
#pragma unroll
          for (int c = 0; c < 8; ++c)
            __stcg(reinterpret_cast<float4*>(mine + ch * 1024 + c * 128), make_float4(z[4 * c], z[4 * c + 1], z[4 * c + 2], z[4 * c + 3]));
        }
        __threadfence();
        __syncwarp();
        int old = 0;
        if (lane == 0) old = atomicAdd(a.counters + (boundary * 2 + rank) * 4 + q, 1);
        old = __shfl_sync(0xffffffffu, old, 0);
        write_out = old == 1;
        if (write_out) __threadfence();
      }
      if (write_out) {
        float4 o[4][8];  // the other cluster's partial, fetched four chunks (half a tile) at a time: the loads of a
                         // lane are independent, and under a loaded memory system each round trip is microseconds
#pragma unroll 1
        for (int ch = 0; ch < chunks; ++ch) {
          if (other != nullptr && (ch & 3) == 0) {
#pragma unroll
            for (int j = 0; j < 4; ++j)
#pragma unroll
              for (int c = 0; c < 8; ++c) o[j][c] = __ldcg(reinterpret_cast<const float4*>(other + (ch + j) * 1024 + c * 128));
          }
          float z[32];
          tc_ld32(t_lane + ch * 32, z);
          tc_wait_ld();
          if (other != nullptr) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              if (j == (ch & 3)) {
#pragma unroll
                for (int c = 0; c < 8; ++c) {
                  z[4 * c] += o[j][c].x;
                  z[4 * c + 1] += o[j][c].y;
                  z[4 * c + 2] += o[j][c].z;
                  z[4 * c + 3] += o[j][c].w;
                }
              }
            }
          }
          if (lane == 0) bulk_wait_read_all();  // the previous block has left the staging memory
          __syncwarp();
          const int sw = (lane >> 1) & 3;
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            uint4 pk;
            pk.x = pack2<OUT>(z[c * 8 + 0], z[c * 8 + 1]);
            pk.y = pack2<OUT>(z[c * 8 + 2], z[c * 8 + 3]);
            pk.z = pack2<OUT>(z[c * 8 + 4], z[c * 8 + 5]);
            pk.w = pack2<OUT>(z[c * 8 + 6], z[c * 8 + 7]);
            *reinterpret_cast<uint4*>(obuf + lane * 64 + ((c ^ sw) << 4)) = pk;
          }
          fence_proxy_async_smem();
          __syncwarp();
          const int col = col0 + ch * 32;
          if (lane == 0 && row0 < a.m && col < a.n) {
            tma_store_2d(&map_c, obuf, col, row0);
            bulk_commit();
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(mapa_u32(smem_u32(&s.tmem_empty[acc]), 0));  // the leader counts both CTAs
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1u;
    }
    if (lane == 0) {
      abort_peer(abort_flag, peer_abort);
      bulk_wait_all();
    }
  }

  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // neither CTA frees tensor memory or exits while the other may still signal it
  tc_fence_after();
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
  }
}

static std::atomic<int> g_gemm_pair{-1};  // -1 = choose per problem, 0 = single-CTA tiles, 1 = CTA pairs

// `inner` contiguous elements x `outer` rows of a 16-bit matrix as boxes of 64 x 64 with the 128-byte swizzle
static bool make_map_mn(CUtensorMap* map, CUtensorMapDataType dt, const void* base, long long inner, long long outer) {
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) return false;
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(inner), static_cast<cuuint64_t>(outer)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(inner) * 2};
  const cuuint32_t box[2] = {64u, 64u}, estr[2] = {1u, 1u};
  return fn(map, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Column sums of a [rows, cols] 16-bit matrix in fp32, two stages, fixed order (dbias = sum of dz over the tokens).
constexpr int kColsumChunks = 64;
template <typename T>
__global__ void __launch_bounds__(128) colsum_stage1(const T* __restrict__ x, float* __restrict__ part, long long rows,
                                                     int cols) {
  // thread -> 8 columns (one 16-byte vector); blockIdx.y -> chunk of rows
  const int v = blockIdx.x * blockDim.x + threadIdx.x;
  if (v * 8 >= cols) return;
  const long long per = (rows + kColsumChunks - 1) / kColsumChunks;
  const long long r0 = blockIdx.y * per, r1 = r0 + per < rows ? r0 + per : rows;
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  for (long long r = r0; r < r1; ++r) {
    Vec<T, 8> w;
    w.load_stream(x + r * cols + v * 8);
    float f[8];
    w.unpack(f);
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] += f[i];
  }
  float* dst = part + static_cast<long long>(blockIdx.y) * cols + v * 8;
#pragma unroll
  for (int i = 0; i < 8; ++i) dst[i] = acc[i];
}
template <typename T>
__global__ void __launch_bounds__(256) colsum_stage2(const float* __restrict__ part, T* __restrict__ out, int cols) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= cols) return;
  float acc = 0.f;
#pragma unroll 8
  for (int k = 0; k < kColsumChunks; ++k) acc += part[static_cast<long long>(k) * cols + c];  // chunks in order
  out[c] = from_f32<T>(acc);
}

}  // namespace nd

// Tuning hook: 1 = two-CTA tiles (cta_group::2, clusters of two CTAs), 0 = single-CTA tiles, negative (the
// default) = choose per problem. Process-wide.
extern "C" void nd_tune_fc1_pair(int mode) { nd::g_fc1_pair.store(mode < 0 ? -1 : (mode != 0 ? 1 : 0)); }

// Diagnostic hook: when set to a device array of 8 int64, later launches add to it, summed over CTAs: [0] cycles
// the copy-issuing thread waited for free stages, [3] cycles one epilogue warp waited for an accumulator, [4]
// cycles that warp spent on tiles, [5] the copy-issuing thread's lifetime in cycles and [7] in nanoseconds (their
// ratio is the SM clock during the launch). The two-CTA kernel reports [5] and [7] only. nullptr turns it off.
// dbias [cols] = sum over `rows` partial rows of part [rows, cols] (fp32), in row order
template <typename T>
__global__ void __launch_bounds__(256) dbias_stage2(const float* __restrict__ part, T* __restrict__ out, int rows, int cols) {
  nd::griddep_wait();
  const int c = blockIdx.x * 256 + threadIdx.x;
  if (c >= cols) return;
  float acc0 = 0.f, acc1 = 0.f, acc2 = 0.f, acc3 = 0.f;  // four interleaved chains, combined in a fixed order
  int r = 0;
  for (; r + 4 <= rows; r += 4) {
    acc0 += part[static_cast<size_t>(r) * cols + c];
    acc1 += part[static_cast<size_t>(r + 1) * cols + c];
    acc2 += part[static_cast<size_t>(r + 2) * cols + c];
    acc3 += part[static_cast<size_t>(r + 3) * cols + c];
  }
  for (; r < rows; ++r) acc0 += part[static_cast<size_t>(r) * cols + c];
  out[c] = nd::from_f32<T>((acc0 + acc1) + (acc2 + acc3));
}

extern "C" void nd_tune_fc1_pdl(int enabled) { nd::g_fc1_pdl.store(enabled != 0 ? 1 : 0); }

extern "C" void nd_tune_fc1_bwd_pair(int mode) { nd::g_gemm_pair.store(mode < 0 ? -1 : (mode != 0 ? 1 : 0)); }

extern "C" void nd_tune_fc1_trace(long long* device_counters) { nd::g_fc1_trace.store(device_counters); }

extern "C" int nd_fc1_fwd(int ab_dtype, int out_dtype, int act, int gated, const void* x, const void* w,
                          const void* bias, float alpha_host, const float* alpha_dev, void* y, int64_t m,
                          int64_t k, int64_t n, int* status, void* stream) {
  using namespace nd;
  if (m < 0 || k <= 0 || n <= 0) return ND_ERR_BAD_ARG;
  if (act != ND_ACT_SILU && act != ND_ACT_GELU && !(act == ND_ACT_NONE && gated == 0)) return ND_ERR_UNSUPPORTED;
  if (out_dtype != ND_BF16 && out_dtype != ND_F16) return ND_ERR_UNSUPPORTED;
  if (ab_dtype != ND_BF16 && ab_dtype != ND_F16 && ab_dtype != ND_E4M3) return ND_ERR_UNSUPPORTED;
  if (gated < 0 || gated > 2) return ND_ERR_BAD_ARG;
  if (gated && (n % 2) != 0) return ND_ERR_BAD_ARG;
  if (m == 0) return ND_OK;
  if (!x || !w || !y) return ND_ERR_BAD_ARG;
  const int es = ab_dtype == ND_E4M3 ? 1 : 2;
  const long long n_out = gated ? n / 2 : n;
  if ((k * es) % 16 != 0 || n_out % 8 != 0) return ND_ERR_UNSUPPORTED;  // TMA row pitch / 16-byte stores
  if (!aligned16(x) || !aligned16(w) || !aligned16(y)) return ND_ERR_UNSUPPORTED;
  if (m > INT32_MAX - kBM || n > INT32_MAX - kBN || k > INT32_MAX - 256) return ND_ERR_UNSUPPORTED;

  Fc1Args a{};
  a.bias = bias; a.y = y; a.alpha_dev = alpha_dev; a.sink = Fc1Sink{status, device_error_ptr()}; a.alpha_host = alpha_host;
  a.trace = g_fc1_trace.load(std::memory_order_relaxed);
  a.m = static_cast<int>(m); a.k = static_cast<int>(k); a.n = static_cast<int>(n);
  a.n_out = static_cast<int>(n_out);
  a.tiles_m = static_cast<int>((m + kBM - 1) / kBM);
  a.tiles_n = static_cast<int>(gated ? (n_out + 127) / 128 : (n + kBN - 1) / kBN);
  a.k_blocks = static_cast<int>((k * es + kBKBytes - 1) / kBKBytes);
  const long long tiles = static_cast<long long>(a.tiles_m) * a.tiles_n;
  if (tiles > INT32_MAX) return ND_ERR_UNSUPPORTED;

  CUtensorMap map_x, map_w;
  const CUtensorMapDataType dt = ab_dtype == ND_E4M3 ? CU_TENSOR_MAP_DATA_TYPE_UINT8
                                 : ab_dtype == ND_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                                       : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  if (!make_map(&map_x, dt, es, x, m, k) || !make_map(&map_w, dt, es, w, n, k)) return ND_ERR_LAUNCH;

  // y as a tensor for the epilogue's block stores: n_out contiguous 16-bit columns, blocks of 32 x 32, 64B swizzle
  CUtensorMap map_y;
  {
    EncodeTiledFn enc = encode_fn();
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(n_out), static_cast<cuuint64_t>(m)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(n_out) * 2};
    const cuuint32_t box[2] = {32u, 32u};
    const cuuint32_t estr[2] = {1u, 1u};
    const CUtensorMapDataType ydt = out_dtype == ND_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    if (enc == nullptr ||
        enc(&map_y, ydt, 2, y, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_64B,
            CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
      return ND_ERR_LAUNCH;
  }

  const int g = gated;
  // Two-CTA tiles halve the B-operand bytes each SM stages and keep the tensor pipe busier per k-block, but the
  // pair's epilogues run in lockstep and a 256-row tile wastes more on small problems: measured faster for
  // 16-bit operands once there are at least two rounds of single-CTA tiles; for FP8 (half the k-blocks per
  // tile, so the epilogue weighs twice as much) slower at K = 1152 (2168 against 2384 TFLOP/s at 8192 x 4608) and
  // faster at K = 3072 (2635 against 2502 at 32768 x 12288): there the pairs start at 16 k-blocks.
  const int pair_mode = g_fc1_pair.load(std::memory_order_relaxed);
  const bool pair = pair_mode >= 0 ? pair_mode != 0
                                   : (tiles >= 2LL * sm_count() && (ab_dtype != ND_E4M3 || a.k_blocks >= 16));
  const void* fn;
  if (pair) {
    if (ab_dtype == ND_E4M3)
      fn = out_dtype == ND_BF16 ? pick_fc1_pair<true, 0, __nv_bfloat16>(act, g) : pick_fc1_pair<true, 0, __half>(act, g);
    else if (ab_dtype == ND_BF16)
      fn = out_dtype == ND_BF16 ? pick_fc1_pair<false, 1, __nv_bfloat16>(act, g) : pick_fc1_pair<false, 1, __half>(act, g);
    else
      fn = out_dtype == ND_BF16 ? pick_fc1_pair<false, 0, __nv_bfloat16>(act, g) : pick_fc1_pair<false, 0, __half>(act, g);
  } else {
    if (ab_dtype == ND_E4M3)
      fn = out_dtype == ND_BF16 ? pick_fc1<true, 0, __nv_bfloat16>(act, g) : pick_fc1<true, 0, __half>(act, g);
    else if (ab_dtype == ND_BF16)
      fn = out_dtype == ND_BF16 ? pick_fc1<false, 1, __nv_bfloat16>(act, g) : pick_fc1<false, 1, __half>(act, g);
    else
      fn = out_dtype == ND_BF16 ? pick_fc1<false, 0, __nv_bfloat16>(act, g) : pick_fc1<false, 0, __half>(act, g);
  }

  const int smem_bytes = static_cast<int>(pair ? sizeof(Fc1PairSmem) : sizeof(Fc1Smem)) + 1024;
  cudaError_t e = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
  if (e != cudaSuccess) {
    set_last_cuda_error(e);
    (void)cudaGetLastError();
    return ND_ERR_LAUNCH;
  }
  void* params[] = {&map_x, &map_w, &map_y, &map_y, &map_y, &a};  // the forward epilogue uses the first output map only
  cudaLaunchConfig_t cfg{};
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = smem_bytes;
  cfg.stream = static_cast<cudaStream_t>(stream);
  // attribute 0: programmatic stream serialization (the kernel's prologue may run while its predecessor in the
  // stream drains; see griddep_wait in the kernels); attribute 1, pairs only: the cluster shape
  cudaLaunchAttribute attrs[2] = {};
  attrs[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attrs[0].val.programmaticStreamSerializationAllowed = g_fc1_pdl.load(std::memory_order_relaxed) != 0 ? 1 : 0;
  cfg.attrs = attrs;
  cfg.numAttrs = 1;
  if (pair) {
    // persistent grid of CTA pairs: as many clusters of two as can be resident, at most one per tile
    cudaLaunchAttribute& attr = attrs[1];
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = 2;
    attr.val.clusterDim.y = 1;
    attr.val.clusterDim.z = 1;
    cfg.numAttrs = 2;
    const long long pair_tiles = static_cast<long long>((a.m + 2 * kBM - 1) / (2 * kBM)) * a.tiles_n;
    cfg.gridDim = dim3(static_cast<unsigned>(2 * (sm_count() / 2)));
    int clusters = 0;
    if (cudaOccupancyMaxActiveClusters(&clusters, fn, &cfg) != cudaSuccess || clusters < 1) {
      (void)cudaGetLastError();
      clusters = sm_count() / 2;
    }
    if (clusters > pair_tiles) clusters = static_cast<int>(pair_tiles);
    cfg.gridDim = dim3(static_cast<unsigned>(2 * clusters));
  } else {
    const long long grid = tiles < sm_count() ? tiles : sm_count();
    cfg.gridDim = dim3(static_cast<unsigned>(grid));
  }
  e = cudaLaunchKernelExC(&cfg, fn, params);
  if (e != cudaSuccess) {
    set_last_cuda_error(e);
    (void)cudaGetLastError();
    return ND_ERR_LAUNCH;
  }
  return ND_OK;
}

// The reference's FC1 backward recomputes z = x W^T + b with F.linear, then differentiates the gated activation in
// eager PyTorch (novadit/ops/fc1_bias_act.py:255-270). Here both happen in ONE launch of the forward kernel's main
// loop with the activation backward as its epilogue: dz [m, n] = [dy * value * act'(gate) | dy * act(gate)] for
// w rows [gate | value]; z never reaches memory. 16-bit operands, single-CTA tiles.
extern "C" size_t nd_fc1_bwd_dbias_ws_bytes(int64_t m, int64_t n) {
  if (m <= 0 || n <= 0) return 0;
  return static_cast<size_t>((m + nd::kBM - 1) / nd::kBM) * 4 * static_cast<size_t>(n) * sizeof(float);
}

static int fc1_bwd_dz_impl(int dtype, int act, const void* x, const void* w, const void* bias, const void* dy, void* dz,
                           void* dbias, void* ws, size_t ws_bytes, int64_t m, int64_t k, int64_t n, int* status,
                           void* stream);

extern "C" int nd_fc1_bwd_dz(int dtype, int act, const void* x, const void* w, const void* bias, const void* dy,
                             void* dz, int64_t m, int64_t k, int64_t n, int* status, void* stream) {
  return fc1_bwd_dz_impl(dtype, act, x, w, bias, dy, dz, nullptr, nullptr, 0, m, k, n, status, stream);
}

extern "C" int nd_fc1_bwd_dz_dbias(int dtype, int act, const void* x, const void* w, const void* bias, const void* dy,
                                   void* dz, void* dbias, void* ws, size_t ws_bytes, int64_t m, int64_t k, int64_t n,
                                   int* status, void* stream) {
  if (!dbias || !ws) return ND_ERR_BAD_ARG;
  return fc1_bwd_dz_impl(dtype, act, x, w, bias, dy, dz, dbias, ws, ws_bytes, m, k, n, status, stream);
}

static int fc1_bwd_dz_impl(int dtype, int act, const void* x, const void* w, const void* bias, const void* dy, void* dz,
                           void* dbias, void* ws, size_t ws_bytes, int64_t m, int64_t k, int64_t n, int* status,
                           void* stream) {
  using namespace nd;
  if (m < 0 || k <= 0 || n <= 0 || (n % 2) != 0) return ND_ERR_BAD_ARG;
  if (act != ND_ACT_SILU && act != ND_ACT_GELU) return ND_ERR_UNSUPPORTED;
  if (dtype != ND_BF16 && dtype != ND_F16) return ND_ERR_UNSUPPORTED;
  if (m == 0) {
    if (dbias != nullptr) {  // no tokens: the sum over them is zero
      cudaError_t ez = cudaMemsetAsync(dbias, 0, static_cast<size_t>(n) * 2, static_cast<cudaStream_t>(stream));
      if (ez != cudaSuccess) {
        set_last_cuda_error(ez);
        (void)cudaGetLastError();
        return ND_ERR_LAUNCH;
      }
    }
    return ND_OK;
  }
  if (!x || !w || !dy || !dz) return ND_ERR_BAD_ARG;
  const long long n_out = n / 2;
  if ((k * 2) % 16 != 0 || n_out % 8 != 0) return ND_ERR_UNSUPPORTED;
  if (!aligned16(x) || !aligned16(w) || !aligned16(dy) || !aligned16(dz)) return ND_ERR_UNSUPPORTED;
  if (m > INT32_MAX - kBM || n > INT32_MAX - kBN || k > INT32_MAX - 256) return ND_ERR_UNSUPPORTED;
  if (dbias != nullptr && ((reinterpret_cast<uintptr_t>(ws) & 15u) != 0 || ws_bytes < nd_fc1_bwd_dbias_ws_bytes(m, n)))
    return ND_ERR_BAD_ARG;

  Fc1Args a{};
  a.dbias_part = dbias != nullptr ? static_cast<float*>(ws) : nullptr;
  a.trace = g_fc1_trace.load(std::memory_order_relaxed);
  a.bias = bias; a.y = dz; a.sink = Fc1Sink{status, device_error_ptr()}; a.alpha_host = 1.f;
  a.m = static_cast<int>(m); a.k = static_cast<int>(k); a.n = static_cast<int>(n);
  a.n_out = static_cast<int>(n_out);
  a.tiles_m = static_cast<int>((m + kBM - 1) / kBM);
  a.tiles_n = static_cast<int>((n_out + 127) / 128);
  a.k_blocks = static_cast<int>((k * 2 + kBKBytes - 1) / kBKBytes);
  const long long tiles = static_cast<long long>(a.tiles_m) * a.tiles_n;
  if (tiles > INT32_MAX) return ND_ERR_UNSUPPORTED;

  const CUtensorMapDataType dt = dtype == ND_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  CUtensorMap map_x, map_w, map_dzg, map_dzv, map_dy;
  if (!make_map(&map_x, dt, 2, x, m, k) || !make_map(&map_w, dt, 2, w, n, k)) return ND_ERR_LAUNCH;
  EncodeTiledFn enc = encode_fn();
  if (enc == nullptr) return ND_ERR_LAUNCH;
  // 32 x 32 blocks, 64-byte swizzle. The two halves of dz are described as separate [m, n_out] tensors with the row
  // pitch of dz, so that a block that hangs over the end of the gate half is clipped instead of reaching into the
  // value half.
  auto block_map = [&](CUtensorMap* map, const void* base, long long cols, long long pitch_elems) {
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(m)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(pitch_elems) * 2};
    const cuuint32_t box[2] = {32u, 32u}, estr[2] = {1u, 1u};
    return enc(map, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
               CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
  };
  const unsigned char* dzb = static_cast<const unsigned char*>(dz);
  if (!block_map(&map_dzg, dzb, n_out, n) || !block_map(&map_dzv, dzb + n_out * 2, n_out, n) ||
      !block_map(&map_dy, dy, n_out, n_out))
    return ND_ERR_LAUNCH;
  // CTA-pair tiles as in the forward pass: once there are at least two rounds of single-CTA tiles
  const int pair_mode = g_fc1_pair.load(std::memory_order_relaxed);
  const bool pair = pair_mode >= 0 ? pair_mode != 0 : tiles >= 2LL * sm_count();
  const void* fn;
  if (pair) {
    if (dtype == ND_BF16)
      fn = act == ND_ACT_SILU ? (const void*)fc1_pair_kernel<false, 1, 1, ND_ACT_SILU, __nv_bfloat16, true>
                              : (const void*)fc1_pair_kernel<false, 1, 1, ND_ACT_GELU, __nv_bfloat16, true>;
    else
      fn = act == ND_ACT_SILU ? (const void*)fc1_pair_kernel<false, 0, 1, ND_ACT_SILU, __half, true>
                              : (const void*)fc1_pair_kernel<false, 0, 1, ND_ACT_GELU, __half, true>;
  } else if (dtype == ND_BF16) {
    fn = act == ND_ACT_SILU ? (const void*)fc1_kernel<false, 1, 1, ND_ACT_SILU, __nv_bfloat16, true>
                            : (const void*)fc1_kernel<false, 1, 1, ND_ACT_GELU, __nv_bfloat16, true>;
  } else {
    fn = act == ND_ACT_SILU ? (const void*)fc1_kernel<false, 0, 1, ND_ACT_SILU, __half, true>
                            : (const void*)fc1_kernel<false, 0, 1, ND_ACT_GELU, __half, true>;
  }
  const int smem_bytes = static_cast<int>(pair ? sizeof(Fc1PairBwdSmem) : sizeof(Fc1BwdSmem)) + 1024;
  cudaError_t e = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
  if (e != cudaSuccess) {
    set_last_cuda_error(e);
    (void)cudaGetLastError();
    return ND_ERR_LAUNCH;
  }
  void* params[] = {&map_x, &map_w, &map_dzg, &map_dzv, &map_dy, &a};
  const long long grid = tiles < sm_count() ? tiles : sm_count();
  {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(static_cast<unsigned>(grid));
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = smem_bytes;
    cfg.stream = static_cast<cudaStream_t>(stream);
    cudaLaunchAttribute attrs[2] = {};
    attrs[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attrs[0].val.programmaticStreamSerializationAllowed = g_fc1_pdl.load(std::memory_order_relaxed) != 0 ? 1 : 0;
    cfg.attrs = attrs;
    cfg.numAttrs = 1;
    if (pair) {  // persistent grid of CTA pairs, as in nd_fc1_fwd
      attrs[1].id = cudaLaunchAttributeClusterDimension;
      attrs[1].val.clusterDim.x = 2;
      attrs[1].val.clusterDim.y = 1;
      attrs[1].val.clusterDim.z = 1;
      cfg.numAttrs = 2;
      const long long pair_tiles = static_cast<long long>((a.m + 2 * kBM - 1) / (2 * kBM)) * a.tiles_n;
      cfg.gridDim = dim3(static_cast<unsigned>(2 * (sm_count() / 2)));
      int clusters = 0;
      if (cudaOccupancyMaxActiveClusters(&clusters, fn, &cfg) != cudaSuccess || clusters < 1) {
        (void)cudaGetLastError();
        clusters = sm_count() / 2;
      }
      if (clusters > pair_tiles) clusters = static_cast<int>(pair_tiles);
      cfg.gridDim = dim3(static_cast<unsigned>(2 * clusters));
    }
    e = cudaLaunchKernelExC(&cfg, fn, params);
  }
  if (e != cudaSuccess) {
    set_last_cuda_error(e);
    (void)cudaGetLastError();
    return ND_ERR_LAUNCH;
  }
  if (dbias != nullptr) {
    const int rows = a.tiles_m * 4, cols = a.n;
    const unsigned blocks = static_cast<unsigned>((cols + 255) / 256);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (dtype == ND_BF16)
      dbias_stage2<__nv_bfloat16><<<blocks, 256, 0, st>>>(a.dbias_part, static_cast<__nv_bfloat16*>(dbias), rows, cols);
    else
      dbias_stage2<__half><<<blocks, 256, 0, st>>>(a.dbias_part, static_cast<__half*>(dbias), rows, cols);
    e = cudaGetLastError();
    if (e != cudaSuccess) {
      set_last_cuda_error(e);
      return ND_ERR_LAUNCH;
    }
  }
  return ND_OK;
}

// The two GEMMs of the FC1 backward on the tcgen05 path, operands read where they lie (no transposes):
//   op 0: c [m, n] = a [m, k] @ b [k, n]      (dx = dz @ W:   m tokens, k = 2I, n = H)
//   op 1: c [m, n] = a [k, m]^T @ b [k, n]    (dW = dz^T @ x: m = 2I, k tokens, n = H)
extern "C" size_t nd_fc1_bwd_gemm_ws_bytes(void) {
  const int pairs = nd::sm_count() / 2;
  return nd::kGpCounterBytes + static_cast<size_t>(pairs > 1 ? pairs - 1 : 0) * 4 * nd::kGpPartialFloats * sizeof(float);
}

extern "C" int nd_fc1_bwd_gemm(int dtype, int op, const void* a, const void* b, void* c, int64_t m, int64_t n, int64_t k,
                               void* ws, size_t ws_bytes, int* status, void* stream) {
  using namespace nd;
  if (m < 0 || n <= 0 || k <= 0) return ND_ERR_BAD_ARG;
  if (dtype != ND_BF16 && dtype != ND_F16) return ND_ERR_UNSUPPORTED;
  if (op != 0 && op != 1) return ND_ERR_BAD_ARG;
  if (m == 0) return ND_OK;
  if (!a || !b || !c) return ND_ERR_BAD_ARG;
  // row pitches of every tensor the copy engine walks must be multiples of 16 bytes
  if (n % 8 != 0 || (op == 0 ? k % 8 != 0 : m % 8 != 0)) return ND_ERR_UNSUPPORTED;
  if (!aligned16(a) || !aligned16(b) || !aligned16(c)) return ND_ERR_UNSUPPORTED;
  if (m > INT32_MAX - kBM || n > INT32_MAX - kGemmBN || k > INT32_MAX - 256) return ND_ERR_UNSUPPORTED;
  GemmArgs g{};
  g.sink = Fc1Sink{status, device_error_ptr()};
  g.m = static_cast<int>(m); g.n = static_cast<int>(n); g.k = static_cast<int>(k);
  g.tiles_m = static_cast<int>((m + kBM - 1) / kBM);
  g.tiles_n = static_cast<int>((n + kGemmBN - 1) / kGemmBN);
  g.k_blocks = static_cast<int>((k + 63) / 64);
  const long long tiles = static_cast<long long>(g.tiles_m) * g.tiles_n;
  if (tiles > INT32_MAX) return ND_ERR_UNSUPPORTED;
  const CUtensorMapDataType dt = dtype == ND_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  CUtensorMap map_a, map_b, map_c;
  const bool ok_a = op == 0 ? make_map(&map_a, dt, 2, a, m, k) : make_map_mn(&map_a, dt, a, m, k);
  if (!ok_a || !make_map_mn(&map_b, dt, b, n, k)) return ND_ERR_LAUNCH;
  {
    EncodeTiledFn enc = encode_fn();
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(n), static_cast<cuuint64_t>(m)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(n) * 2};
    const cuuint32_t box[2] = {32u, 32u}, estr[2] = {1u, 1u};
    if (enc == nullptr ||
        enc(&map_c, dt, 2, c, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_64B,
            CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
      return ND_ERR_LAUNCH;
  }
  const int pair_mode = g_gemm_pair.load();
  const bool ws_ok = ws != nullptr && (reinterpret_cast<uintptr_t>(ws) & 255u) == 0 && ws_bytes >= nd_fc1_bwd_gemm_ws_bytes();
  // Whole 128 x 192 tiles waste the empty part of their last round over the SMs and the overhang of the last column
  // tile; the evenly cut pair tiles waste only the overhang of the last 256-wide column tile (whose MMAs cost as much
  // as a full tile's). Take the pairs where that is the smaller loss by a margin (measured: equal at 8192 x 1152,
  // 8 - 15 % faster at 1024 / 1280 columns, 5 % slower where whole tiles already fill their rounds).
  bool use_pairs = pair_mode == 1;
  if (pair_mode < 0 && m > kBM) {
    const long long rounds = (tiles + sm_count() - 1) / sm_count();
    const double fill_single = static_cast<double>(tiles) / static_cast<double>(rounds * sm_count()) *
                               static_cast<double>(n) / static_cast<double>(g.tiles_n * static_cast<long long>(kGemmBN));
    const double fill_pair = static_cast<double>(n) / static_cast<double>(((n + 255) / 256) * 256);
    use_pairs = fill_pair > 1.03 * fill_single;
  }
  if (ws_ok && sm_count() >= 4 && use_pairs) {
    GemmPairArgs gp{};
    gp.sink = g.sink;
    gp.trace = g_fc1_trace.load(std::memory_order_relaxed);
    gp.counters = static_cast<int*>(ws);
    gp.partials = reinterpret_cast<float*>(static_cast<uint8_t*>(ws) + kGpCounterBytes);
    gp.m = g.m; gp.n = g.n; gp.k = g.k;
    gp.tiles_n = static_cast<int>((n + 255) / 256);
    gp.k_blocks = g.k_blocks;
    const long long pair_tiles = ((m + 2 * kBM - 1) / (2 * kBM)) * gp.tiles_n;
    gp.total_it = pair_tiles * gp.k_blocks;
    const void* fnp;
    if (dtype == ND_BF16)
      fnp = op == 0 ? (const void*)gemm_bwd_pair_kernel<1, false, __nv_bfloat16>
                    : (const void*)gemm_bwd_pair_kernel<1, true, __nv_bfloat16>;
    else
      fnp = op == 0 ? (const void*)gemm_bwd_pair_kernel<0, false, __half> : (const void*)gemm_bwd_pair_kernel<0, true, __half>;
    const int smem_pair = static_cast<int>(sizeof(GemmPairSmem)) + 1024;
    cudaError_t ep = cudaFuncSetAttribute(fnp, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_pair);
    if (ep != cudaSuccess) {
      set_last_cuda_error(ep);
      (void)cudaGetLastError();
      return ND_ERR_LAUNCH;
    }
    void* pp[] = {&map_a, &map_b, &map_c, &gp};
    cudaLaunchConfig_t pc{};
    pc.blockDim = dim3(kGemmThreads);
    pc.dynamicSmemBytes = smem_pair;
    pc.stream = static_cast<cudaStream_t>(stream);
    cudaLaunchAttribute attr{};
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = 2;
    attr.val.clusterDim.y = 1;
    attr.val.clusterDim.z = 1;
    pc.attrs = &attr;
    pc.numAttrs = 1;
    pc.gridDim = dim3(static_cast<unsigned>(2 * (sm_count() / 2)));
    int clusters = 0;
    if (cudaOccupancyMaxActiveClusters(&clusters, fnp, &pc) != cudaSuccess || clusters < 1) {
      (void)cudaGetLastError();
      clusters = sm_count() / 2;
    }
    if (clusters > sm_count() / 2) clusters = sm_count() / 2;   // the workspace is sized for that many
    if (clusters > pair_tiles) clusters = static_cast<int>(pair_tiles);  // a range is at least one tile long
    pc.gridDim = dim3(static_cast<unsigned>(2 * clusters));
    ep = cudaMemsetAsync(ws, 0, kGpCounterBytes, pc.stream);
    if (ep == cudaSuccess) ep = cudaLaunchKernelExC(&pc, fnp, pp);
    if (ep != cudaSuccess) {
      set_last_cuda_error(ep);
      (void)cudaGetLastError();
      return ND_ERR_LAUNCH;
    }
    return ND_OK;
  }
  const void* fn;
  if (dtype == ND_BF16)
    fn = op == 0 ? (const void*)gemm_bwd_kernel<1, false, __nv_bfloat16> : (const void*)gemm_bwd_kernel<1, true, __nv_bfloat16>;
  else
    fn = op == 0 ? (const void*)gemm_bwd_kernel<0, false, __half> : (const void*)gemm_bwd_kernel<0, true, __half>;
  const int smem_bytes = static_cast<int>(sizeof(GemmSmem)) + 1024;
  cudaError_t e = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
  if (e != cudaSuccess) {
    set_last_cuda_error(e);
    (void)cudaGetLastError();
    return ND_ERR_LAUNCH;
  }
  void* params[] = {&map_a, &map_b, &map_c, &g};
  cudaLaunchConfig_t cfg{};
  cfg.blockDim = dim3(kGemmThreads);
  cfg.dynamicSmemBytes = smem_bytes;
  cfg.stream = static_cast<cudaStream_t>(stream);
  cfg.gridDim = dim3(static_cast<unsigned>(tiles < sm_count() ? tiles : sm_count()));
  cudaLaunchAttribute pdl{};
  pdl.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  pdl.val.programmaticStreamSerializationAllowed = g_fc1_pdl.load(std::memory_order_relaxed) != 0 ? 1 : 0;
  cfg.attrs = &pdl;
  cfg.numAttrs = 1;
  e = cudaLaunchKernelExC(&cfg, fn, params);
  if (e != cudaSuccess) {
    set_last_cuda_error(e);
    (void)cudaGetLastError();
    return ND_ERR_LAUNCH;
  }
  return ND_OK;
}

extern "C" size_t nd_colsum_ws_bytes(int64_t cols) {
  return cols > 0 ? static_cast<size_t>(nd::kColsumChunks) * cols * sizeof(float) : 0;
}

// out [cols] = column sums of x [rows, cols] (16-bit; cols a multiple of 8), fp32 accumulation in a fixed order
extern "C" int nd_colsum(int dtype, const void* x, int64_t rows, int64_t cols, void* out, void* ws, size_t ws_bytes,
                         void* stream) {
  using namespace nd;
  if (rows < 0 || cols <= 0) return ND_ERR_BAD_ARG;
  if (dtype != ND_BF16 && dtype != ND_F16) return ND_ERR_UNSUPPORTED;
  if (cols % 8 != 0 || cols > INT32_MAX || !aligned16(x)) return ND_ERR_UNSUPPORTED;
  if (!x || !out) return ND_ERR_BAD_ARG;
  if (!ws || ws_bytes < nd_colsum_ws_bytes(cols) || (reinterpret_cast<uintptr_t>(ws) & 15u)) return ND_ERR_WORKSPACE;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const dim3 g1(static_cast<unsigned>((cols / 8 + 127) / 128), kColsumChunks);
  const unsigned g2 = static_cast<unsigned>((cols + 255) / 256);
  float* part = static_cast<float*>(ws);
  if (dtype == ND_BF16) {
    colsum_stage1<__nv_bfloat16><<<g1, 128, 0, st>>>(static_cast<const __nv_bfloat16*>(x), part, rows, static_cast<int>(cols));
    colsum_stage2<__nv_bfloat16><<<g2, 256, 0, st>>>(part, static_cast<__nv_bfloat16*>(out), static_cast<int>(cols));
  } else {
    colsum_stage1<__half><<<g1, 128, 0, st>>>(static_cast<const __half*>(x), part, rows, static_cast<int>(cols));
    colsum_stage2<__half><<<g2, 256, 0, st>>>(part, static_cast<__half*>(out), static_cast<int>(cols));
  }
  return check_launch();
}
