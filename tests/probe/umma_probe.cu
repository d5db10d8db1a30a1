// Test-only library (libtriattn_probe.so): one tcgen05 MMA tile from caller-built shared-memory operand
// images, D[128 x n] = A . B^T.  The parity tests use it to pin the operand-layout conventions of the prefill
// kernels (128-byte-swizzled A rows, 128-byte core-matrix blobs for B) against plain integer / float products.
// It is not part of the product ABI and nothing in the package loads it.
//
// The entry point refuses, without launching, any request that is not one of the operand shapes the kernels
// use: instruction descriptors come from a fixed list, layouts are "none" or "128-byte swizzle", and every byte
// a descriptor can address must lie inside the image that was copied to shared memory.
#include "tcgen05.cuh"
#include "abi_internal.h"
#include <cstdio>

namespace tri {

constexpr int ProbeThreads = 128;
constexpr int ProbeImage = 32768;   // bytes reserved per operand image

__global__ void __launch_bounds__(ProbeThreads) umma_probe_kernel(const uint8_t* a_img, int a_bytes, const uint8_t* b_img,
    int b_bytes, uint32_t a_lbo, uint32_t a_sbo, uint32_t a_layout, uint32_t a_step, uint32_t b_lbo, uint32_t b_sbo,
    uint32_t b_layout, uint32_t b_step, uint32_t idesc, int f16_kind, int ksteps, int ncols, uint32_t* out, int* err) {
  extern __shared__ uint8_t raw_smem[];
  __shared__ __align__(8) uint64_t bar;
  __shared__ uint32_t tmem_slot;
  uint8_t* smem = raw_smem + ((1024u - (smem_u32(raw_smem) & 1023u)) & 1023u);
  const int tid = threadIdx.x, warp = tid / 32;
  for (int i = tid; i < a_bytes / 16; i += ProbeThreads) reinterpret_cast<uint4*>(smem)[i] = reinterpret_cast<const uint4*>(a_img)[i];
  for (int i = tid; i < b_bytes / 16; i += ProbeThreads)
    reinterpret_cast<uint4*>(smem + ProbeImage)[i] = reinterpret_cast<const uint4*>(b_img)[i];
  if (tid == 0) { mbar_init(&bar, 1); mbar_fence_init(); }
  if (warp == 0) { tmem_alloc(&tmem_slot, 256); tmem_relinquish(); }
  fence_proxy_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_slot;
  if (tid == 0) {
    const uint32_t aa = smem_u32(smem), ba = smem_u32(smem + ProbeImage);
    for (int kk = 0; kk < ksteps; ++kk) {
      const uint64_t ad = smem_desc(aa + kk * a_step, a_lbo, a_sbo, a_layout), bd = smem_desc(ba + kk * b_step, b_lbo, b_sbo, b_layout);
      if (f16_kind) umma_f16(tmem, ad, bd, idesc, kk > 0);
      else umma_i8(tmem, ad, bd, idesc, kk > 0);
    }
    tc_commit(&bar);
  }
  __syncwarp();
  bool ok = mbar_wait(&bar, 0);
  ok = __syncthreads_and(ok);
  if (ok) {
    tc_fence_after();
    for (int c = 0; c < ncols / 16; ++c) {
      uint32_t a[16];
      tmem_ld16(tmem + ((uint32_t)(warp * 32) << 16) + c * 16, a);
      tmem_ld_wait();
#pragma unroll
      for (int j = 0; j < 16; ++j) out[(int64_t)tid * ncols + c * 16 + j] = a[j];
    }
  } else if (tid == 0) {
    atomicExch(err, ErrBarrierTimeout);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, 256);
}

// Last byte (exclusive) that `ksteps` MMAs with 32 bytes of K each can read from an operand of `rows` rows.
static int64_t addressed_extent(int rows, uint32_t lbo, uint32_t sbo, uint32_t layout, uint32_t step, int ksteps) {
  const int64_t last_start = (int64_t)(ksteps - 1) * step;
  // 128-byte swizzle: an atom is 8 rows x 128 B and a K step moves inside the row, so only whole rows count
  if (layout == Layout128B) return (last_start & ~(int64_t)127) + (int64_t)(rows / 8 - 1) * sbo + 1024;
  return last_start + (int64_t)(rows / 8 - 1) * sbo + lbo + 128;                         // two 128-byte core matrices along K
}

}  // namespace tri

using namespace tri;

static thread_local char g_probe_error[256] = "";
void tri_set_error(const char* what) { snprintf(g_probe_error, sizeof g_probe_error, "%s", what); }
int tri_launch_status(const char* where) {
  const cudaError_t e = cudaGetLastError();
  if (e == cudaSuccess) return TRI_OK;
  snprintf(g_probe_error, sizeof g_probe_error, "%s: %s", where, cudaGetErrorString(e));
  return TRI_ERR_CUDA;
}

extern "C" const char* tri_probe_last_error(void) { return g_probe_error; }

extern "C" int tri_umma_probe(const void* a_img, int a_bytes, const void* b_img, int b_bytes, uint32_t a_lbo, uint32_t a_sbo,
    uint32_t a_layout, uint32_t a_step, uint32_t b_lbo, uint32_t b_sbo, uint32_t b_layout, uint32_t b_step, uint32_t idesc,
    int f16_kind, int ksteps, int ncols, uint32_t* out, int* device_error, void* stream) {
  TRI_CHECK(a_img && b_img && out && device_error, "umma_probe: null buffers");
  TRI_CHECK(a_bytes > 0 && a_bytes <= ProbeImage && b_bytes > 0 && b_bytes <= ProbeImage && a_bytes % 16 == 0 &&
            b_bytes % 16 == 0 && ksteps > 0 && ksteps <= 8, "umma_probe: sizes");
  // the operand shapes of the kernels: (descriptor, fp16/bf16 kind?, accumulator columns)
  struct Shape { uint32_t idesc; int f16; int n; };
  const Shape known[] = {{IdescQK, 0, 64}, {IdescPV16, 1, 128}, {IdescBias, 1, 64},
                         {instr_desc(2, 0, 1, 128, 128), 0, 128},    // u8 x s8 -> s32 (integer P.V)
                         {instr_desc(1, 1, 1, 128, 64), 1, 64},      // bf16 x bf16 -> f32 (un-quantised scores)
                         {instr_desc(1, 1, 1, 128, 128), 1, 128}};   // bf16 x bf16 -> f32 (un-quantised P.V)
  bool listed = false;
  for (const Shape& s : known) listed |= s.idesc == idesc && s.f16 == (f16_kind != 0) && s.n == ncols;
  TRI_CHECK(listed, "umma_probe: instruction descriptor / kind / width is not one the kernels use");
  TRI_CHECK((a_layout == LayoutNone || a_layout == Layout128B) && (b_layout == LayoutNone || b_layout == Layout128B),
            "umma_probe: layout type");
  TRI_CHECK(a_lbo % 16 == 0 && a_sbo % 16 == 0 && b_lbo % 16 == 0 && b_sbo % 16 == 0 && a_step % 16 == 0 && b_step % 16 == 0 &&
            a_lbo < (1u << 18) && a_sbo < (1u << 18) && b_lbo < (1u << 18) && b_sbo < (1u << 18), "umma_probe: offsets");
  TRI_CHECK(addressed_extent(128, a_lbo, a_sbo, a_layout, a_step, ksteps) <= a_bytes &&
            addressed_extent(ncols, b_lbo, b_sbo, b_layout, b_step, ksteps) <= b_bytes,
            "umma_probe: a descriptor addresses bytes outside its operand image");
  static TriPerDevice configured;
  const int device = configured.pending();
  TRI_CHECK(device != -2, "umma_probe: no current CUDA device");
  if (device >= 0) {
    TRI_CUDA(cudaFuncSetAttribute(umma_probe_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 2 * ProbeImage + 1024), "probe");
    configured.mark(device);
  }
  umma_probe_kernel<<<1, ProbeThreads, 2 * ProbeImage + 1024, static_cast<cudaStream_t>(stream)>>>(static_cast<const uint8_t*>(a_img),
      a_bytes, static_cast<const uint8_t*>(b_img), b_bytes, a_lbo, a_sbo, a_layout, a_step, b_lbo, b_sbo, b_layout, b_step, idesc,
      f16_kind, ksteps, ncols, out, device_error);
  return tri_launch_status("umma_probe");
}
