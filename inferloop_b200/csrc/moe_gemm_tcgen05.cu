// Grouped bfloat16 matrix product on the tcgen05 tensor cores: the experts of a routed
// feed-forward over rows that are sorted by expert.
//
//     out[rows of block b, :] = A[rows of block b, :] * W[group[b]]^T        (block = 128 or 256 rows)
//
// A is [rows, K] with every block of rows belonging to one group (csrc/moe.cu deals the
// rows), W is [groups, N, K], group[b] < 0 marks a block that holds no rows and is skipped.
// One CTA computes one tile: D accumulates in tensor memory over K; warp 0 (one lane) streams
// the operands by TMA (cp.async.bulk.tensor, 128-byte swizzle, no multicast) through a ring of
// three stages, warp 1 (one lane) issues tcgen05.mma and commits, warps 2-5 read the
// accumulators with tcgen05.ld and write the rows out.  Tile shapes: 128 rows x 128 weight
// rows, two CTAs to an SM so that one tile's write-out runs under the other's products (few
// rows per expert: the launch streams the chosen experts' weights); 128 x 256 with a ring of four
// stages, one tile a CTA or (the default for many rows) persistent CTAs with two accumulators;
// and 256 x 256 (two 128-row accumulators that share every weight block, all 512 columns of
// tensor memory): wider tiles need fewer operand bytes per flop.  The weight tile of group
// g starts at row g * N + n0 of the stacked matrix; columns past N are not written, so a tile
// that reaches into the next group's rows (or past the end, where TMA fills zeros) is harmless.
// With the SwiGLU epilogue W holds blocks of 64 gate rows followed by their 64 up rows, a tile is
// one such pair, and out[:, n0/2 .. n0/2 + 63] = silu(gate) * up, so the [rows, 2 I] intermediate
// is never written.  Every mbarrier wait is bounded; on expiry the kernel raises the error flag,
// lets its other warps leave their waits, frees its tensor memory and returns.
#include <cuda.h>
#include <mutex>
#include <unordered_map>
#include "common.cuh"
#include "sm100.cuh"

using namespace ilb;

namespace {

constexpr int kBlockK = 64;             // bf16 elements per K block = one 128-byte swizzle row
constexpr int kRows = 128;              // rows of one accumulator = MMA M
constexpr uint32_t kBytesA = kRows * kBlockK * 2;
// MS row blocks of 128 and BN weight rows per tile
template <int MS, int BN> __host__ __device__ constexpr uint32_t stage_bytes() { return MS * kBytesA + BN * kBlockK * 2; }
template <int MS, int BN, int kStages> constexpr size_t smem_bytes() { return (size_t)kStages * stage_bytes<MS, BN>() + 1024 + (2 * kStages + 4) * 8; }


// K-major operand tile, 128-byte swizzle: rows of 128 bytes, 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr) {
  return (uint64_t)((addr & 0x3FFFFu) >> 4) | (1ull << 16) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
// D = 32-bit, A and B = bfloat16, both K-major.
__host__ __device__ constexpr uint32_t instr_desc(int mma_m, int mma_n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(mma_n >> 3) << 17) | ((uint32_t)(mma_m >> 4) << 24);
}

struct Params {
  void* out;                 // [rows, N] (SwiGLU: [rows, N / 2]), bf16 or f32
  const int* block_group;    // [rows / rows of a tile]
  int* error_flag;
  int N, K, ldo, k_blocks;
  int swiglu, out_f32;
  // the gated unit of the epilogue: a(g) * (u + act_offset), a(g) = g * sigmoid(act_sharp * g), with g = min(gate, act_limit)
  // and u = clamp(up, -act_limit, act_limit) when act_limit > 0 (sharpness 1, no limit, offset 0: silu(gate) * up)
  float act_limit, act_sharp, act_offset;
};

__device__ __forceinline__ float glu_mul(const Params& p, float g, float u) {
  if (p.act_limit > 0.f) { g = fminf(g, p.act_limit); u = fminf(fmaxf(u, -p.act_limit), p.act_limit); }
  return __fdividef(g, 1.0f + __expf(-p.act_sharp * g)) * (u + p.act_offset);
}

// 32 consecutive columns of one output row, from column c on; columns from `limit` on are not written.
__device__ __forceinline__ void store32(const Params& p, size_t out_row, int c, int limit, const float (&v)[32]) {
  if (p.out_f32) {
    float* o = (float*)p.out + out_row + c;
    if (c + 32 <= limit && p.ldo % 4 == 0 && ((uintptr_t)p.out % 16 == 0)) {
#pragma unroll
      for (int j = 0; j < 32; j += 4) *reinterpret_cast<float4*>(o + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j) if (c + j < limit) o[j] = v[j];
    }
  } else {
    __nv_bfloat16* o = (__nv_bfloat16*)p.out + out_row + c;
    if (c + 32 <= limit && p.ldo % 8 == 0 && ((uintptr_t)p.out % 16 == 0)) {
#pragma unroll
      for (int j = 0; j < 32; j += 8)
        *reinterpret_cast<uint4*>(o + j) = make_uint4(pack_bf16(v[j], v[j + 1]), pack_bf16(v[j + 2], v[j + 3]),
                                                      pack_bf16(v[j + 4], v[j + 5]), pack_bf16(v[j + 6], v[j + 7]));
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j) if (c + j < limit) o[j] = __float2bfloat16_rn(v[j]);
    }
  }
}

template <int MS, int BN, int kStages>
__global__ void __launch_bounds__(192, (MS == 1 && BN == 128) ? 2 : 1)
moe_gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w, const Params p) {
  constexpr uint32_t kStageBytes = stage_bytes<MS, BN>();
  constexpr uint32_t kTmemCols = MS * BN;          // 128 or 512: a power of two
  pdl_launch_dependents();
  pdl_wait();                                    // the rows and their groups are the preceding kernels' work
  const int b = blockIdx.y;
  const int g = p.block_group[b];
  if (g < 0) return;                             // (the whole CTA, before anything is set up)
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (base - smem_u32(smem_raw));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kStages * kStageBytes);
  const uint32_t full0 = smem_u32(bars), empty0 = full0 + 8 * kStages, tfull = empty0 + 8 * kStages;
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(bars + 2 * kStages + 1);
  volatile int* failed = reinterpret_cast<volatile int*>(bars + 2 * kStages + 2);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = blockIdx.x * BN;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 1); }
    mbar_init(tfull, 1);
    *failed = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32((const void*)tmem_slot)), "r"(kTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {                             // ---- TMA producer
      bool ok = true;
      for (int it = 0; it < p.k_blocks; ++it) {
        const uint32_t s = it % kStages;
        if (it >= kStages) {
          ok = mbar_wait(empty0 + 8 * s, ((it / kStages) - 1) & 1);
          if (!ok) break;
        }
        const uint32_t dst = base + s * kStageBytes;
        mbar_expect_tx(full0 + 8 * s, kStageBytes);
#pragma unroll
        for (int ms = 0; ms < MS; ++ms) tma_load_2d(dst + ms * kBytesA, &map_a, full0 + 8 * s, it * kBlockK, (b * MS + ms) * kRows);
        tma_load_2d(dst + MS * kBytesA, &map_w, full0 + 8 * s, it * kBlockK, g * p.N + n0);
      }
      if (!ok) { *failed = 1; if (p.error_flag) *p.error_flag = 1; }
    }
  } else if (warp == 1) {
    if (lane == 0) {                             // ---- MMA issuer
      constexpr uint32_t idesc = instr_desc(kRows, BN);
      bool ok = true;
      for (int it = 0; it < p.k_blocks; ++it) {
        const uint32_t s = it % kStages;
        ok = mbar_wait(full0 + 8 * s, (it / kStages) & 1);
        if (!ok) break;
        tcgen05_fence_after();
        const uint32_t a = base + s * kStageBytes;
        const uint64_t db = smem_desc(a + MS * kBytesA);
#pragma unroll
        for (int ms = 0; ms < MS; ++ms) {
          const uint64_t da = smem_desc(a + ms * kBytesA);
#pragma unroll
          for (int k = 0; k < kBlockK / 16; ++k) mma_bf16(tmem_base + ms * BN, da + 2 * k, db + 2 * k, idesc, (it > 0 || k > 0) ? 1u : 0u);
        }
        tcgen05_commit(empty0 + 8 * s);          // the stage is free once these products have read it
      }
      if (!ok) { *failed = 1; if (p.error_flag) *p.error_flag = 1; }
      tcgen05_commit(tfull);                     // arrives when every product issued so far is complete
    }
  } else {
    // ---- write-out: warps 2..5 own tensor-memory lanes 32 (warp & 3) .. + 31, one row each
    const int quad = warp & 3;
    const int row = quad * 32 + lane;
    if (!mbar_wait(tfull, 0)) { *failed = 1; if (p.error_flag) *p.error_flag = 1; }
    tcgen05_fence_after();
    if (*failed == 0) {
#pragma unroll 1
      for (int ms = 0; ms < MS; ++ms) {
        const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + ms * BN;
        const size_t out_row = (size_t)((b * MS + ms) * kRows + row) * p.ldo;
        if (p.swiglu) {
          // a pair of 64 gate rows and their 64 up rows gives 64 output columns
#pragma unroll 1
          for (int pair = 0; pair < BN / 128; ++pair) {
#pragma unroll
            for (int half = 0; half < 2; ++half) {
              const int c = n0 / 2 + pair * 64 + 32 * half;
              if (c >= p.N / 2) continue;
              float gt[32], up[32];
              tmem_load_32(taddr + pair * 128 + 32 * half, gt);
              tmem_load_32(taddr + pair * 128 + 64 + 32 * half, up);
              float v[32];
#pragma unroll
              for (int j = 0; j < 32; ++j) v[j] = glu_mul(p, gt[j], up[j]);
              store32(p, out_row, c, p.N / 2, v);
            }
          }
        } else {
#pragma unroll 1
          for (int c0 = 0; c0 < BN; c0 += 32) {
            const int c = n0 + c0;
            if (c >= p.N) break;
            float v[32];
            tmem_load_32(taddr + c0, v);
            store32(p, out_row, c, p.N, v);
          }
        }
      }
    }
  }
  tcgen05_fence_before();
  __syncthreads();
  if (warp == 1) {
    tcgen05_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
  }
}

// The same product with persistent CTAs, for launches of many tiles: one CTA an SM walks the
// tiles blockIdx.x, blockIdx.x + gridDim.x, ... (weight tiles of a block of rows are neighbours, so
// CTAs that run side by side share the rows' operand in L2), the operand ring runs on across the
// tiles, and two accumulators of BN columns take turns: a tile is written out while the next one
// is multiplied.  The blocks that hold rows are the first ones (csrc/moe.cu fills them in expert
// order), so a CTA is done at the first block without a group.
template <int BN, int kStages>
__global__ void __launch_bounds__(192, 1)
moe_gemm_persistent_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w, const Params p,
                           int n_blocks, int tiles_n) {
  constexpr uint32_t kStageBytes = stage_bytes<1, BN>();
  constexpr uint32_t kTmemCols = 2 * BN;           // 512 for BN = 256
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (base - smem_u32(smem_raw));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kStages * kStageBytes);
  const uint32_t full0 = smem_u32(bars), empty0 = full0 + 8 * kStages, tfull0 = empty0 + 8 * kStages, tempty0 = tfull0 + 16;
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(bars + 2 * kStages + 4);
  volatile int* failed = reinterpret_cast<volatile int*>(bars + 2 * kStages + 5);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long total = (long long)n_blocks * tiles_n;
  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(tfull0 + 8 * b, 1); mbar_init(tempty0 + 8 * b, 128); }
    *failed = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32((const void*)tmem_slot)), "r"(kTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // the tile after `t` of this CTA, or false when there is none
  auto tile_at = [&](long long t, int& b, int& n0, int& g) {
    if (t >= total) return false;
    b = (int)(t / tiles_n);
    n0 = (int)(t % tiles_n) * BN;
    g = __ldg(p.block_group + b);
    return g >= 0;
  };

  if (warp == 0) {
    if (lane == 0) {                             // ---- TMA producer
      bool ok = true;
      uint32_t it = 0;
      int b, n0, g;
      for (long long t = blockIdx.x; ok && tile_at(t, b, n0, g); t += gridDim.x) {
        for (int kb = 0; kb < p.k_blocks; ++kb, ++it) {
          const uint32_t s = it % kStages;
          if (it >= (uint32_t)kStages) {
            ok = mbar_wait(empty0 + 8 * s, ((it / kStages) - 1) & 1);
            if (!ok) break;
          }
          const uint32_t dst = base + s * kStageBytes;
          mbar_expect_tx(full0 + 8 * s, kStageBytes);
          tma_load_2d(dst, &map_a, full0 + 8 * s, kb * kBlockK, b * kRows);
          tma_load_2d(dst + kBytesA, &map_w, full0 + 8 * s, kb * kBlockK, g * p.N + n0);
        }
      }
      if (!ok) { *failed = 1; if (p.error_flag) *p.error_flag = 1; }
    }
  } else if (warp == 1) {
    if (lane == 0) {                             // ---- MMA issuer
      constexpr uint32_t idesc = instr_desc(kRows, BN);
      bool ok = true;
      uint32_t it = 0, j = 0;
      int b, n0, g;
      for (long long t = blockIdx.x; ok && tile_at(t, b, n0, g); t += gridDim.x, ++j) {
        const uint32_t buf = j & 1;
        ok = mbar_wait(tempty0 + 8 * buf, ((j >> 1) & 1) ^ 1);     // the write-out has drained this accumulator
        if (!ok) break;
        tcgen05_fence_after();
        for (int kb = 0; kb < p.k_blocks; ++kb, ++it) {
          const uint32_t s = it % kStages;
          ok = mbar_wait(full0 + 8 * s, (it / kStages) & 1);
          if (!ok) break;
          tcgen05_fence_after();
          const uint32_t a = base + s * kStageBytes;
          const uint64_t da = smem_desc(a), db = smem_desc(a + kBytesA);
#pragma unroll
          for (int k = 0; k < kBlockK / 16; ++k) mma_bf16(tmem_base + buf * BN, da + 2 * k, db + 2 * k, idesc, (kb > 0 || k > 0) ? 1u : 0u);
          tcgen05_commit(empty0 + 8 * s);
        }
        if (ok) tcgen05_commit(tfull0 + 8 * buf);
      }
      if (!ok) {
        *failed = 1; if (p.error_flag) *p.error_flag = 1;
        tcgen05_commit(tfull0); tcgen05_commit(tfull0 + 8);       // let the write-out leave its wait
      }
    }
  } else {
    // ---- write-out: warps 2..5 own tensor-memory lanes 32 (warp & 3) .. + 31, one row each
    const int quad = warp & 3;
    const int row = quad * 32 + lane;
    uint32_t j = 0;
    int b, n0, g;
    for (long long t = blockIdx.x; tile_at(t, b, n0, g); t += gridDim.x, ++j) {
      const uint32_t buf = j & 1;
      if (!mbar_wait(tfull0 + 8 * buf, (j >> 1) & 1)) { *failed = 1; if (p.error_flag) *p.error_flag = 1; }
      tcgen05_fence_after();
      if (*failed != 0) break;
      const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + buf * BN;
      const size_t out_row = (size_t)(b * kRows + row) * p.ldo;
      if (p.swiglu) {
#pragma unroll 1
        for (int pair = 0; pair < BN / 128; ++pair) {
#pragma unroll
          for (int half = 0; half < 2; ++half) {
            const int c = n0 / 2 + pair * 64 + 32 * half;
            if (c >= p.N / 2) continue;
            float gt[32], up[32];
            tmem_load_32(taddr + pair * 128 + 32 * half, gt);
            tmem_load_32(taddr + pair * 128 + 64 + 32 * half, up);
            float v[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = glu_mul(p, gt[i], up[i]);
            store32(p, out_row, c, p.N / 2, v);
          }
        }
      } else {
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += 32) {
          const int c = n0 + c0;
          if (c >= p.N) break;
          float v[32];
          tmem_load_32(taddr + c0, v);
          store32(p, out_row, c, p.N, v);
        }
      }
      tcgen05_fence_before();
      mbar_arrive(tempty0 + 8 * buf);            // the accumulator may be written again
    }
  }
  tcgen05_fence_before();
  __syncthreads();
  if (warp == 1) {
    tcgen05_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
  }
}

struct MapKey {
  const void* ptr; long long rows; int cols, ld, box_rows;
  bool operator==(const MapKey& o) const { return ptr == o.ptr && rows == o.rows && cols == o.cols && ld == o.ld && box_rows == o.box_rows; }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    size_t h = std::hash<const void*>()(k.ptr) * 1000003u ^ std::hash<long long>()(k.rows);
    for (int v : {k.cols, k.ld, k.box_rows}) h = h * 1000003u ^ std::hash<int>()(v);
    return h;
  }
};

// A [rows, cols] bf16 matrix with leading dimension ld (elements); box = [box_rows, 64].
int make_map(CUtensorMap* out, const void* ptr, long long rows, int cols, int ld, int box_rows) {
  static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
  static std::mutex mu;
  const MapKey key{ptr, rows, cols, ld, box_rows};
  std::lock_guard<std::mutex> guard(mu);
  auto it = cache.find(key);
  if (it != cache.end()) { *out = it->second; return 0; }
  EncodeTiledFn fn = encode_fn();
  if (!fn) return fail("moe_gemm: cuTensorMapEncodeTiled is not available from this driver");
  const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  const cuuint32_t box[2] = {(cuuint32_t)kBlockK, (cuuint32_t)box_rows};
  const cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail("moe_gemm: cuTensorMapEncodeTiled failed with code %d (rows %lld cols %d ld %d)", (int)r, rows, cols, ld);
  if (cache.size() > 4096) cache.clear();
  cache.emplace(key, *out);
  return 0;
}

}  // namespace

template <int MS, int BN, int kStages>
static int launch_tiles(const void* A, const void* W, const Params& p, int rows, int groups, int lda, cudaStream_t stream) {
  static OncePerDevice once;
  constexpr size_t smem = smem_bytes<MS, BN, kStages>();
  if (once.first() &&
      cudaFuncSetAttribute(moe_gemm_kernel<MS, BN, kStages>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
    once.forget();
    return fail("moe_gemm: cannot reserve %zu bytes of shared memory", smem);
  }
  CUtensorMap ma, mw;
  if (make_map(&ma, A, rows, p.K, lda, kRows)) return -1;
  if (make_map(&mw, W, (long long)groups * p.N, p.K, p.K, BN)) return -1;
  ilb::launch(moe_gemm_kernel<MS, BN, kStages>, dim3((p.N + BN - 1) / BN, rows / (MS * kRows)), dim3(192), smem, stream, ma, mw, p);
  return check_launch("moe_gemm_tc");
}

template <int BN, int kStages>
static int launch_persistent(const void* A, const void* W, const Params& p, int rows, int groups, int lda, cudaStream_t stream) {
  static OncePerDevice once;
  constexpr size_t smem = smem_bytes<1, BN, kStages>() + 64;
  if (once.first() &&
      cudaFuncSetAttribute(moe_gemm_persistent_kernel<BN, kStages>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
    once.forget();
    return fail("moe_gemm: cannot reserve %zu bytes of shared memory", smem);
  }
  CUtensorMap ma, mw;
  if (make_map(&ma, A, rows, p.K, lda, kRows)) return -1;
  if (make_map(&mw, W, (long long)groups * p.N, p.K, p.K, BN)) return -1;
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 148;
  const int n_blocks = rows / kRows, tiles_n = (p.N + BN - 1) / BN;
  const long long total = (long long)n_blocks * tiles_n;
  ilb::launch(moe_gemm_persistent_kernel<BN, kStages>, dim3((unsigned)(total < sms ? total : sms)), dim3(192), smem, stream, ma, mw, p,
              n_blocks, tiles_n);
  return check_launch("moe_gemm_tc");
}

// Whether these sizes meet the TMA rules (rows of 16 bytes, 16-byte bases).
ILB_EXPORT int ilb_moe_gemm_tc_supported(int N, int K, int lda, int swiglu) {
  return (K % 8 == 0 && lda % 8 == 0 && N > 0 && (!swiglu || N % 128 == 0)) ? 1 : 0;
}

// A: [rows, K] bf16 (leading dimension lda); W: [groups, N, K] bf16, contiguous; out: [rows, N]
// (with swiglu: [rows, N / 2]) bf16 or f32 with leading dimension ldo; block_group: [rows / block_rows],
// block_rows = 128 or 256; tile_n = 128 or 256 weight rows per tile (256 rows take 256); tile_n = 257
// asks for the persistent form of the 128 x 256 tile.
ILB_EXPORT int ilb_moe_gemm_tc(const void* A, const void* W, void* out, int out_f32, int rows, int groups, int N, int K, int lda,
                               int ldo, int swiglu, const int* block_group, int block_rows, int tile_n, int* error_flag,
                               float act_limit, float act_sharp, float act_offset, cudaStream_t stream) {
  ILB_REQUIRE(rows >= 0 && groups > 0 && N > 0 && K > 0, "moe_gemm: bad sizes rows=%d groups=%d N=%d K=%d", rows, groups, N, K);
  ILB_REQUIRE(block_rows == 128 || block_rows == 256, "moe_gemm: blocks of 128 or 256 rows, not %d", block_rows);
  ILB_REQUIRE(tile_n == 256 || ((tile_n == 128 || tile_n == 257) && block_rows == 128), "moe_gemm: tiles of %d x %d are not built", block_rows, tile_n);
  ILB_REQUIRE(rows % block_rows == 0 && rows / block_rows <= 65535, "moe_gemm: rows must come in blocks of %d (at most 65535 blocks)", block_rows);
  ILB_REQUIRE(K % 8 == 0 && lda % 8 == 0 && lda >= K && ((uintptr_t)A % 16 == 0) && ((uintptr_t)W % 16 == 0),
              "moe_gemm: operands must have rows of whole 16 bytes on 16-byte boundaries");
  ILB_REQUIRE(!swiglu || N % 128 == 0, "moe_gemm: the SwiGLU epilogue needs gate and up rows in blocks of 64");
  ILB_REQUIRE(ldo >= (swiglu ? N / 2 : N), "moe_gemm: output rows too short");
  ILB_REQUIRE(block_group != nullptr, "moe_gemm: needs the group of every block of rows");
  ILB_REQUIRE((long long)groups * N < 2147483647LL, "moe_gemm: too many weight rows");
  if (rows == 0) return 0;
  Params p;
  p.out = out; p.block_group = block_group; p.error_flag = error_flag;
  p.N = N; p.K = K; p.ldo = ldo; p.k_blocks = (K + kBlockK - 1) / kBlockK;
  p.swiglu = swiglu ? 1 : 0; p.out_f32 = out_f32 ? 1 : 0;
  p.act_limit = act_limit; p.act_sharp = act_sharp; p.act_offset = act_offset;
  if (block_rows == 256) return launch_tiles<2, 256, 3>(A, W, p, rows, groups, lda, stream);
  if (tile_n == 257) return launch_persistent<256, 4>(A, W, p, rows, groups, lda, stream);
  if (tile_n == 256) return launch_tiles<1, 256, 4>(A, W, p, rows, groups, lda, stream);
  return launch_tiles<1, 128, 3>(A, W, p, rows, groups, lda, stream);
}

ILB_DEFINE_LAST_ERROR()
