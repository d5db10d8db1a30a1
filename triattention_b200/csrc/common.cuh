// Shared constants, layouts and PTX wrappers for the sm_100a quantised-attention kernels.
//
// Numerics follow the reference's CUDA sources (paths inside the reference project):
//   triattention/kernels/cuda/prefill_sm80.cu:14-28,78-115  constants, P rounding, dither, rotation
//   triattention/kernels/cuda/common_device.cuh             quantise / statistics / decode arithmetic
// The whole library is compiled with --use_fast_math like the reference
// (triattention/kernels/extension.py:52) so that `/`, `1/x` and exp2f lower to the same hardware
// approximations and scale bit patterns agree.
//
// HBM tile layouts ("blobs") used by every kernel here.  A tile is 64 keys of one KV head.
// All blobs are sequences of 128-byte core matrices (8 rows x 16 bytes), the canonical no-swizzle
// K-major shared-memory layout of tcgen05.mma, which is also conflict-free for mma.sync B-fragment
// reads (a warp reads one whole core matrix per 32-bit load).
//   K8  8192 B  [key/8][feature/16][key%8][feature%16]            int8
//   K4X 8192 B  same as K8, holding the 4-bit codes as int8        (prefill operand only)
//   K4  4096 B  [key/8][key%8][sub=feature/32][16 B]; word s, byte j: low nibble = feature
//               32*sub+8s+j, high nibble = feature 32*sub+8s+4+j   (decode cache layout, see decode_kernel.cuh)
//   V8  8192 B  [ch/8][key/16][ch%8][16 B]; byte 4s+b = key 16*blk + kperm(s,b)
//   V4  4096 B  [ch/8][kc=key/32][ch%8][16 B]; byte 4s+b: low nibble = key 32kc+kperm(s,b),
//               high nibble = key 32kc+16+kperm(s,b)
//   V16 16384 B [ch/8][key/8][ch%8][key%8]                         fp16, natural key order
// kperm(s,b) = 2s + (b<2 ? b : b+6) is the order in which an mma.sync accumulator lane holds the
// keys of a 16-key group (the reference uses the same permutation, prefill_sm80.cu:93).
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <math_constants.h>
#include <cfloat>
#include <cstdint>

namespace tri {

constexpr int D = 128;            // head dimension (prefill_sm80.cu:14)
constexpr int BN = 64;            // keys per tile
constexpr int BM = 64;            // query rows per query block
constexpr int StatBlocks = 64;    // common_device.cuh:30
constexpr int MaxGroup = 8;       // common_device.cuh:174
constexpr int MaxTiles = 2048;    // 131072 tokens (prefill_sm80.cu:23,518)
constexpr int Magic = 0x4B400000; // 12582912.0f (prefill_sm80.cu:27)
constexpr int K8Bytes = 8192, K4Bytes = 4096, V8Bytes = 8192, V4Bytes = 4096, V16Bytes = 16384;
constexpr int StatFloats = 3 * D;

__host__ __device__ __forceinline__ int kperm(int s, int b) { return 2 * s + (b < 2 ? b : b + 6); }

// ---- error word shared by kernels with bounded waits ----------------------------------------
// Kernels never trap or spin forever: a wait that runs out records a code here and the CTA leaves.
enum DeviceError : int { ErrNone = 0, ErrBarrierTimeout = 1, ErrTmemAlloc = 2, ErrBadTask = 3, ErrBadSlot = 4 };

// ---- rotation (prefill_sm80.cu:95-115) --------------------------------------------------------
__device__ __constant__ uint32_t kRotationSigns[4] = {0x9a3b5e71u, 0x2c6d8f13u, 0xe41b7a95u, 0x5f02c3d8u};
constexpr float kRotScale = 0.08838834764831845f;

// Reference thread mapping: lane holds features 4*lane..4*lane+3 of one row, a warp holds a row.
__device__ __forceinline__ void rotate128_x4(float (&x)[4], int lane) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int c = lane * 4 + i;
    if ((kRotationSigns[c >> 5] >> (c & 31)) & 1u) x[i] = -x[i];
  }
  const float a = x[0] + x[1], b = x[0] - x[1], c2 = x[2] + x[3], d = x[2] - x[3];
  x[0] = a + c2; x[1] = b + d; x[2] = a - c2; x[3] = b - d;
#pragma unroll
  for (int bit = 1; bit < 32; bit <<= 1) {
    const bool upper = lane & bit;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float y = __shfl_xor_sync(0xffffffffu, x[i], bit);
      x[i] = upper ? y - x[i] : x[i] + y;
    }
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) x[i] *= kRotScale;
}

// Same butterflies (feature bits 0..6 in order, lower = lo+hi, upper = lo-hi, one final multiply)
// with 16 features per lane and 8 lanes per row: four in-register stages, three shuffle stages.
// l8 = lane%8 selects features 16*l8..16*l8+15.  Bit-identical to rotate128_x4 per element.
__device__ __forceinline__ void rotate128_x16(float (&x)[16], int l8) {
  const uint32_t mask = (kRotationSigns[l8 >> 1] >> (16 * (l8 & 1))) & 0xffffu;
#pragma unroll
  for (int i = 0; i < 16; ++i) if ((mask >> i) & 1u) x[i] = -x[i];
#pragma unroll
  for (int bit = 1; bit < 16; bit <<= 1) {
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      if (!(i & bit)) {
        const float lo = x[i], hi = x[i | bit];
        x[i] = lo + hi; x[i | bit] = lo - hi;
      }
    }
  }
#pragma unroll
  for (int bit = 1; bit < 8; bit <<= 1) {
    const float sign = (l8 & bit) ? -1.f : 1.f;   // upper lane: partner - own; lower lane: own + partner
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const float y = __shfl_xor_sync(0xffffffffu, x[i], bit);
      x[i] = fmaf(x[i], sign, y);                 // one rounding of y +- x, like the add / subtract it replaces
    }
  }
#pragma unroll
  for (int i = 0; i < 16; ++i) x[i] *= kRotScale;
}

// ---- P quantisation helpers (prefill_sm80.cu:78-88,255-257) -----------------------------------
constexpr float PMagicHalf = 49152.5f;
__device__ __forceinline__ float pmagic_dither(int acc_bits) {
  return __int_as_float((acc_bits & 0xff) | 0x47400000);
}
__device__ __forceinline__ uint32_t pack_bytes(uint32_t w0, uint32_t w1, uint32_t w2, uint32_t w3) {
  return __byte_perm(__byte_perm(w0, w1, 0x0051), __byte_perm(w2, w3, 0x0051), 0x5410);
}
__device__ __forceinline__ float tile_base_margin(float slope, float base) {
  return fmaf(slope, 0.75f, fabsf(base) * 2.4e-7f);
}

// ---- mbarrier / bulk-copy (TMA) wrappers -------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
  return ok != 0;
}
// Programmatic dependent launch: a kernel launched with launch_chained() (host side) may become resident
// while the kernel before it in the stream still runs.  grid_dependency_wait() returns once that kernel
// has completed and its writes are visible (a no-op for a plain launch), so everything that reads the
// predecessor's results or overwrites what it reads sits behind it; grid_launch_dependents() lets the
// next kernel of the stream start its own prologue.
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void grid_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// Bounded wait: gives up after `limit_ns` of wall time (read from %globaltimer every 64 polls) and
// returns false.  The caller records ErrBarrierTimeout and leaves; nothing spins forever.
__device__ __forceinline__ uint64_t globaltimer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, uint64_t limit_ns = 2000000000ull) {
  if (mbar_try_wait(bar, parity)) return true;
  const uint64_t t0 = globaltimer_ns();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 64; ++i)
      if (mbar_try_wait(bar, parity)) return true;
    if (globaltimer_ns() - t0 > limit_ns) return false;
  }
}
// Bounded, abortable wait for kernels whose warps wait on different barriers: gives up when the CTA's
// abort flag (shared memory) is set by anyone, or sets it itself after ~2 s.  After an abort every warp
// keeps following its control flow without computing, so no thread is left behind at a barrier.
__device__ __forceinline__ bool mbar_wait_abortable(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  if (mbar_try_wait(bar, parity)) return true;
  const uint64_t t0 = globaltimer_ns();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 32; ++i)
      if (mbar_try_wait(bar, parity)) return true;
    if (*abort_flag) return false;
    if (globaltimer_ns() - t0 > 2000000000ull) { *abort_flag = 1; return false; }
  }
}
// The same with the waiting done by the hardware: try_wait with a suspend-time hint parks the warp until
// the phase completes or the hint (in ns) runs out, so a warp that waits issues one instruction per ~20 us
// instead of a polling loop that competes with working warps for issue slots.
__device__ __forceinline__ bool mbar_try_wait_parked(uint64_t* bar, uint32_t parity, uint32_t ns) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity), "r"(ns) : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool mbar_wait_parked(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int site = 1) {
  if (mbar_try_wait_parked(bar, parity, 20000u)) return true;
  if (*abort_flag) return false;   // after an abort nothing completes any more: every later wait costs one try
  const uint64_t t0 = globaltimer_ns();
  for (;;) {
    // the hardware usually hands the warp back long before the hint runs out: the abort flag and the clock are looked
    // at once per eight tries, so that a waiting warp costs the working ones few issue slots
#pragma unroll 1
    for (int i = 0; i < 8; ++i)
      if (mbar_try_wait_parked(bar, parity, 20000u)) return true;
    if (*abort_flag) return false;
    if (globaltimer_ns() - t0 > 2000000000ull) { *abort_flag = site; return false; }   // site != 0: tells which wait gave up
  }
}
// 1-D bulk copy global -> shared; dst, src and bytes are multiples of 16.
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// ---- legacy warp MMA used by the (HBM-bound) decode kernel ------------------------------------
__device__ __forceinline__ void mma_s8(int (&c)[4], uint32_t a0, uint32_t a2, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3]) : "r"(a0), "r"(0u), "r"(a2), "r"(0u), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mma_u8s8(int (&c)[4], uint32_t a0, uint32_t a2, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3]) : "r"(a0), "r"(0u), "r"(a2), "r"(0u), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], uint32_t a0, uint32_t a2, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(0u), "r"(a2), "r"(0u), "r"(b0), "r"(b1));
}

}  // namespace tri
