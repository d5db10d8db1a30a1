// Measurement-only kernel (part of libtriattn_probe.so): what the tcgen05 INT8 path sustains on this GPU when it
// does nothing but multiply.  One CTA per SM issues back-to-back kind::i8 MMAs of shape M128 N256 K32 from operands
// resident in shared memory (A: 128 rows x 128 B with the 128-byte swizzle, B: 256 rows as 128-byte core matrices;
// the operand conventions of the prefill kernel, at the widest N), alternating between two 256-column accumulators
// in tensor memory.  bench.py times it with CUDA events and reports the prefill's tensor throughput against it,
// beside the nominal figure.  Nothing in the package uses it.
#include "tcgen05.cuh"
#include "abi_internal.h"

namespace tri {

constexpr int PeakThreads = 128;
constexpr int PeakABytes = 16384, PeakBBytes = 32768;           // 4 K-steps of 32 bytes each
constexpr int PeakShared = PeakABytes + PeakBBytes + 1024;

__global__ void __launch_bounds__(PeakThreads, 1) i8_peak_kernel(int iterations, int* err) {
  extern __shared__ uint8_t raw_smem[];
  __shared__ __align__(8) uint64_t bar;
  __shared__ uint32_t tmem_slot;
  uint8_t* smem = raw_smem + ((1024u - (smem_u32(raw_smem) & 1023u)) & 1023u);
  const int tid = threadIdx.x, warp = tid / 32;
  // operand bytes: a cheap hash, so that the multipliers see switching data like real codes
  for (int i = tid; i < (PeakABytes + PeakBBytes) / 4; i += PeakThreads) {
    uint32_t x = (uint32_t)i * 2654435761u + blockIdx.x * 40503u;
    x ^= x >> 15; x *= 2246822519u; x ^= x >> 13;
    reinterpret_cast<uint32_t*>(smem)[i] = x;
  }
  if (tid == 0) { mbar_init(&bar, 1); mbar_fence_init(); }
  if (warp == 0) { tmem_alloc(&tmem_slot, 512); tmem_relinquish(); }
  fence_proxy_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_slot;
  constexpr uint32_t idesc = instr_desc(2, 1, 1, 128, 256);   // s8 x s8 -> s32, M128 N256
  if (tid == 0) {
    const uint64_t da = smem_desc(smem_u32(smem), 0, 1024, Layout128B);
    const uint64_t db = smem_desc(smem_u32(smem + PeakABytes), 128, 1024, LayoutNone);
    for (int it = 0; it < iterations; ++it) {
      const uint32_t d = tmem + (uint32_t)(it & 1) * 256;
#pragma unroll
      for (int kk = 0; kk < 4; ++kk)
        umma_i8(d, da + (uint64_t)((kk * 32) >> 4), db + (uint64_t)((kk * 256) >> 4), idesc, (it > 1 || kk > 0) ? 1u : 0u);
    }
    tc_commit(&bar);
  }
  __syncwarp();
  bool ok = mbar_wait(&bar, 0, 4000000000ull);   // bounded: gives up after 4 s
  ok = __syncthreads_and(ok);
  if (!ok && tid == 0) atomicExch(err, ErrBarrierTimeout);
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, 512);
}

}  // namespace tri

using namespace tri;

// Launches `ctas` CTAs that each issue iterations x 4 MMAs (M128 N256 K32).  Returns the operations one CTA performs
// (2 * 128 * 256 * 32 per MMA) through ops_per_cta (host pointer), so that the caller's arithmetic cannot drift from
// the kernel's shape.
extern "C" int tri_i8_peak(int ctas, int iterations, int64_t* ops_per_cta, int* device_error, void* stream) {
  TRI_CHECK(ctas > 0 && ctas <= 4096 && iterations > 0 && iterations <= (1 << 22) && ops_per_cta && device_error, "i8_peak: arguments");
  static TriPerDevice configured;
  const int device = configured.pending();
  TRI_CHECK(device != -2, "i8_peak: no current CUDA device");
  if (device >= 0) {
    TRI_CUDA(cudaFuncSetAttribute(i8_peak_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, PeakShared), "i8_peak");
    configured.mark(device);
  }
  *ops_per_cta = (int64_t)iterations * 4 * 2 * 128 * 256 * 32;
  i8_peak_kernel<<<ctas, PeakThreads, PeakShared, static_cast<cudaStream_t>(stream)>>>(iterations, device_error);
  return tri_launch_status("i8_peak");
}
