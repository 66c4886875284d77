// Fused FC1: y = epilogue((x @ w^T) * alpha + bias) on the 5th-generation tensor cores (sm_100a).
//
// One persistent CTA per SM, 320 threads, warp-specialised:
//   warp 0      TMA producer: x and w tiles -> 128B-swizzled shared memory, 4-stage mbarrier ring
//   warp 1      tcgen05.mma issuer (one lane) + owner of the tensor-memory allocation
//   warps 2..9  epilogue (two warps per TMEM lane quarter, each taking half of the tile's columns):
//               tcgen05.ld the fp32 accumulator, * alpha, + bias, activation
//               (gated: value * act(gate)), round once, 64-byte row segments to global memory
// CTA tile: 128 rows x 256 accumulator columns x 128 bytes of K per stage. For the gated form
// the 256 columns are 128 gate columns and the 128 value columns of the SAME output columns,
// staged as one K-major B operand (gate rows then value rows), so a single UMMA of N=256
// produces both halves and the epilogue combines TMEM columns c and 128+c. Two accumulators
// (2 x 256 of the 512 TMEM columns) let the epilogue of tile i overlap the main loop of tile
// i+1. No cluster, no multicast: every CTA issues its own TMA loads.
//
// Every wait on an mbarrier is bounded (1 s of %globaltimer); on expiry the waiting role raises
// a CTA-wide abort flag, the status word in global memory is set, every role leaves its loop,
// the producer lets its copies in flight land, and tensor memory is freed before the CTA exits.
#include <cuda.h>
#include <cuda_fp8.h>

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
constexpr int kGroupM = 8;       // tile rasterisation: m-blocks per group
constexpr unsigned long long kWaitLimitNs = 1000000000ull;

struct Fc1Args {
  const void* bias;        // out dtype, length n (nullable)
  void* y;
  const float* alpha_dev;  // nullable, two floats multiplied into alpha
  int* status;             // nullable
  float alpha_host;
  int m, k, n;             // n = rows of w
  int n_out;               // columns of y (n/2 gated, n plain)
  int tiles_m, tiles_n, k_blocks;
};

struct __align__(1024) Fc1Smem {
  uint8_t stage[kStages][kStageBytes];
  float bias[kEpilogueWarps][kBN];  // one private copy per epilogue warp: no cross-warp barrier in the epilogue
  uint64_t full[kStages];
  uint64_t empty[kStages];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint32_t tmem_base;
  int abort_flag;
};

// Bounded wait. Returns false if the CTA is aborting or the limit expired (and raises the abort).
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag,
                                          int* status, int code) {
  if (mbar_try_wait(bar, parity)) return true;
  const unsigned long long t0 = global_ns();
  for (uint32_t polls = 1;; ++polls) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((polls & 255u) == 0) {
      if (*abort_flag) return false;
      if (global_ns() - t0 > kWaitLimitNs) {
        *abort_flag = 1;
        if (status != nullptr) atomicCAS(status, 0, code);
        return false;
      }
    }
  }
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

__device__ __forceinline__ void tc_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}

template <bool F8>
__device__ __forceinline__ void tc_mma(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                       uint32_t accumulate) {
  if constexpr (F8) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
  } else {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
  }
}

// 32 consecutive fp32 columns of this thread's TMEM lane
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

// ABF: instruction-descriptor operand format (kind::f16: 0 = f16, 1 = bf16; kind::f8f6f4: 0 = e4m3)
// GATED: 0 = y = act(z); 1 = w rows [gate block | value block]; 2 = w rows interleaved (gate0, value0, gate1, ...)
template <bool F8, int ABF, int GATED, int ACT, typename OUT>
__global__ void __launch_bounds__(kThreads, 1)
fc1_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
           const Fc1Args a) {
  extern __shared__ uint8_t smem_raw[];
  Fc1Smem& s = *reinterpret_cast<Fc1Smem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  volatile int* abort_flag = &s.abort_flag;
  constexpr int kBKElems = F8 ? 128 : 64;
  const int total_tiles = a.tiles_m * a.tiles_n;

  if (threadIdx.x == 0) {
    for (int i = 0; i < kStages; ++i) {
      mbar_init(&s.full[i], 1);
      mbar_init(&s.empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&s.tmem_full[i], 1);
      mbar_init(&s.tmem_empty[i], kEpilogueWarps);
    }
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

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer
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
        ok = __all_sync(0xffffffffu, mbar_wait(&s.empty[stage], phase ^ 1u, abort_flag, a.status, 1));
        if (!ok) break;
        if (lane == 0) {
          mbar_expect_tx(&s.full[stage], kStageBytes);
          uint8_t* base = s.stage[stage];
          tma_load_2d(base, &map_x, &s.full[stage], kb * kBKElems, m0);
          tma_load_2d(base + kATileBytes, &map_w, &s.full[stage], kb * kBKElems, nb0);
          tma_load_2d(base + kATileBytes + kBHalfBytes, &map_w, &s.full[stage], kb * kBKElems, nb1);
        }
        __syncwarp();
        if (++stage == kStages) {
          stage = 0;
          phase ^= 1u;
        }
      }
    }
    if (!ok) {
      // let copies already issued land in shared memory before the CTA may exit
      const unsigned long long t0 = global_ns();
      while (global_ns() - t0 < 200000ull) __nanosleep(1000);
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    int stage = 0;
    uint32_t phase = 0;
    int acc = 0;
    uint32_t acc_phase = 0;
    constexpr uint32_t idesc = umma_idesc(ABF);
    bool ok = true;
    for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
      ok = __all_sync(0xffffffffu, mbar_wait(&s.tmem_empty[acc], acc_phase ^ 1u, abort_flag, a.status, 2));
      if (!ok) break;
      tc_fence_after();
      const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * kBN);
      for (int kb = 0; kb < a.k_blocks; ++kb) {
        ok = __all_sync(0xffffffffu, mbar_wait(&s.full[stage], phase, abort_flag, a.status, 3));
        if (!ok) break;
        tc_fence_after();
        if (lane == 0) {
          const uint32_t a_addr = smem_u32(s.stage[stage]);
          const uint64_t da = umma_desc(a_addr);
          const uint64_t db = umma_desc(a_addr + kATileBytes);
#pragma unroll
          for (int kk = 0; kk < kBKBytes / 32; ++kk) {
            // advance 32 bytes of K inside the swizzle span: +2 in 16-byte address units
            tc_mma<F8>(d_tmem, da + 2ull * kk, db + 2ull * kk, idesc, (kb | kk) != 0 ? 1u : 0u);
          }
          tc_commit(&s.empty[stage]);  // the stage is free again once these MMAs have read it
        }
        __syncwarp();
        if (++stage == kStages) {
          stage = 0;
          phase ^= 1u;
        }
      }
      if (!ok) break;
      if (lane == 0) tc_commit(&s.tmem_full[acc]);
      __syncwarp();
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1u;
    }
  } else {
    // ---------------------------------------------------------------- epilogue (4 warps)
    const int q = warp & 3;             // TMEM lane quarter this warp may read
    const int colhalf = (warp - 2) >> 2;   // which half of the tile's column steps this warp takes
    int acc = 0;
    uint32_t acc_phase = 0;
    float alpha = a.alpha_host;
    if (a.alpha_dev != nullptr) alpha *= __ldg(a.alpha_dev) * __ldg(a.alpha_dev + 1);
    const OUT* __restrict__ bias = static_cast<const OUT*>(a.bias);
    OUT* __restrict__ y = static_cast<OUT*>(a.y);
    bool ok = true;
    for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
      int mi, ni;
      tile_coords(a, t, mi, ni);
      const int out0 = GATED != 0 ? ni * 128 : ni * kBN;  // first output column of the tile
      // bias of the tile's 256 accumulator columns -> this warp's shared-memory copy (fp32)
      float* sb = s.bias[warp - 2];
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
      ok = __all_sync(0xffffffffu, mbar_wait(&s.tmem_full[acc], acc_phase, abort_flag, a.status, 4));
      if (!ok) break;
      tc_fence_after();
      const int row = mi * kBM + q * 32 + lane;
      const uint32_t t_lane = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + static_cast<uint32_t>(acc * kBN);
      // per step: kOutPer output columns of this thread's row (a whole number of 16-byte stores)
      constexpr int kSteps = GATED == 1 ? 4 : 8;
      constexpr int kOutPer = GATED == 2 ? 16 : 32;
#pragma unroll 1
      for (int ch = colhalf * (kSteps / 2); ch < (colhalf + 1) * (kSteps / 2); ++ch) {
        float out[kOutPer];
        if constexpr (GATED == 1) {
          float g[32], v[32];
          tc_ld32(t_lane + ch * 32, g);
          tc_ld32(t_lane + 128 + ch * 32, v);
          tc_wait_ld();
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const float zg = fmaf(g[j], alpha, sb[ch * 32 + j]);
            const float zv = fmaf(v[j], alpha, sb[128 + ch * 32 + j]);
            out[j] = zv * act_fwd<ACT>(zg);
          }
        } else if constexpr (GATED == 2) {
          float z[32];
          tc_ld32(t_lane + ch * 32, z);
          tc_wait_ld();
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const float zg = fmaf(z[2 * j], alpha, sb[ch * 32 + 2 * j]);
            const float zv = fmaf(z[2 * j + 1], alpha, sb[ch * 32 + 2 * j + 1]);
            out[j] = zv * act_fwd<ACT>(zg);
          }
        } else {
          float z[32];
          tc_ld32(t_lane + ch * 32, z);
          tc_wait_ld();
#pragma unroll
          for (int j = 0; j < 32; ++j) out[j] = act_fwd<ACT>(fmaf(z[j], alpha, sb[ch * 32 + j]));
        }
        if (row < a.m) {
          OUT* dst = y + static_cast<long long>(row) * a.n_out + out0 + ch * kOutPer;
#pragma unroll
          for (int v8 = 0; v8 < kOutPer / 8; ++v8) {
            if (out0 + ch * kOutPer + v8 * 8 < a.n_out) {  // n_out is a multiple of 8
              uint4 pk;
              pk.x = pack2<OUT>(out[v8 * 8 + 0], out[v8 * 8 + 1]);
              pk.y = pack2<OUT>(out[v8 * 8 + 2], out[v8 * 8 + 3]);
              pk.z = pack2<OUT>(out[v8 * 8 + 4], out[v8 * 8 + 5]);
              pk.w = pack2<OUT>(out[v8 * 8 + 6], out[v8 * 8 + 7]);
              *reinterpret_cast<uint4*>(dst + v8 * 8) = pk;
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&s.tmem_empty[acc]);
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1u;
    }
  }

  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
  }
}

// ------------------------------------------------------------------ host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
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
      return silu ? (const void*)fc1_kernel<F8, ABF, 0, ND_ACT_SILU, OUT> : (const void*)fc1_kernel<F8, ABF, 0, ND_ACT_GELU, OUT>;
  }
}

}  // namespace nd

extern "C" int nd_fc1_fwd(int ab_dtype, int out_dtype, int act, int gated, const void* x, const void* w,
                          const void* bias, float alpha_host, const float* alpha_dev, void* y, int64_t m,
                          int64_t k, int64_t n, int* status, void* stream) {
  using namespace nd;
  if (m < 0 || k <= 0 || n <= 0) return ND_ERR_BAD_ARG;
  if (act != ND_ACT_SILU && act != ND_ACT_GELU) return ND_ERR_UNSUPPORTED;
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
  a.bias = bias; a.y = y; a.alpha_dev = alpha_dev; a.status = status; a.alpha_host = alpha_host;
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

  const void* fn;
  const int g = gated;
  if (ab_dtype == ND_E4M3)
    fn = out_dtype == ND_BF16 ? pick_fc1<true, 0, __nv_bfloat16>(act, g) : pick_fc1<true, 0, __half>(act, g);
  else if (ab_dtype == ND_BF16)
    fn = out_dtype == ND_BF16 ? pick_fc1<false, 1, __nv_bfloat16>(act, g) : pick_fc1<false, 1, __half>(act, g);
  else
    fn = out_dtype == ND_BF16 ? pick_fc1<false, 0, __nv_bfloat16>(act, g) : pick_fc1<false, 0, __half>(act, g);

  const int smem_bytes = static_cast<int>(sizeof(Fc1Smem)) + 1024;
  cudaError_t e = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
  if (e != cudaSuccess) {
    set_last_cuda_error(e);
    (void)cudaGetLastError();
    return ND_ERR_LAUNCH;
  }
  const long long grid = tiles < sm_count() ? tiles : sm_count();
  void* params[] = {&map_x, &map_w, &a};
  e = cudaLaunchKernel(fn, dim3(static_cast<unsigned>(grid)), dim3(kThreads), params, smem_bytes,
                       static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) {
    set_last_cuda_error(e);
    (void)cudaGetLastError();
    return ND_ERR_LAUNCH;
  }
  return ND_OK;
}
