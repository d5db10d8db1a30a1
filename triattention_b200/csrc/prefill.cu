// Banded causal prefill attention on tcgen05 (sm_100a): INT8 QK^T and INT8 / FP16 PV as dense
// tensor-core contractions with TMEM accumulators.
//
// Replaces (paths inside the reference project)
//   triattention/kernels/cuda/prefill_sm80.cu:158-257  qk8 / qk4 fragments, masks, scaled row max, margin
//   triattention/kernels/cuda/prefill_sm80.cu:259-488  run_task: tile lists, passes, online softmax, epilogue
//   triattention/kernels/cuda/prefill_sm80.cu:490-543  unified_kernel, attention() host launcher
// in band mode (the only mode the reference's Python ever uses, kernels/prefill.py:103), with a batch
// dimension added.
//
// Shape of the computation: see prefill_kernel.cuh (one CTA per 256 query rows of a Q head, warp
// specialised: TMA producer, MMA issuer, softmax).  The two 128-row MMA tiles of a CTA are made
// of four 64-row query blocks that follow the reference's tile lists (sink tile, own diagonal tile, INT8
// band, INT4 band); a tile that only some blocks visit runs with the other blocks' weights at zero.
// INT4 QK uses the 4-bit codes widened to int8 by the write kernel (K4X blobs, Q4X rows), so the
// integer accumulators equal the reference's s4 x s4 MMAs exactly.
// Q arrives by TMA tensor copies (cp.async.bulk.tensor, 128-byte swizzle), K/V tiles by TMA bulk
// copies of pre-tiled blobs (cp.async.bulk).  Every wait is bounded.
#include "tcgen05.cuh"
#include "abi_internal.h"
#include <type_traits>

namespace tri {

// ---- shared-memory / tensor-memory plan of the prefill CTA ------------------------------------
constexpr int RowSplit = 2;           // softmax threads per query row (1 or 2; measured on config 3: 4.84 ms with 2, 5.60 ms with 1)
constexpr int PrefillThreads = (4 + 8 * RowSplit) * 32;   // producer, 2 QK^T issuers, P.V issuer, 8 * RowSplit softmax warps
constexpr int ProbeThreads = 128;   // qk_accum_kernel
constexpr int MaxSteps = 2 * MaxTiles + 8;
constexpr int SmQ8 = 0, SmQ4 = 32768;                            // 2 Q tiles each
constexpr int SmBiasA = 65536, SmBiasB = SmBiasA + 4096;         // constant fp16 operands of the bias MMA (see IdescBias)
constexpr int SmK = SmBiasB + 2048 + 2048;                       // four stages of K (1024-byte aligned)
constexpr int SmV16 = SmK + 4 * K8Bytes, SmEnd = SmV16 + 2 * V16Bytes;   // two fp16 V operands
constexpr int SmSteps = SmEnd, StepBytes = (3 * MaxSteps + 15) / 16 * 16;  // visiting order: uint16 tile|mode, uint8 mask
constexpr int ListBytes = 2 * 4 * MaxSteps;                     // per MMA tile: one word per step it takes part in
constexpr int PrefillShared = SmSteps + StepBytes + ListBytes + 1024;   // + slack to align the base to 1024 bytes
constexpr uint32_t TmemCols = 512, TmemO = 0, TmemS = 256;      // O: [tile] x 128 columns; S: [tile][buffer] x 64
constexpr float RefSlack = 8.f;   // a row's reference exponent moves when a tile's maximum exceeds it by this (log2)
constexpr float PMagic64 = 58368.5f;   // 2^15 * 1.78125 + 0.5: like 49152.5f, with 0x64 in byte 2 of the sum
constexpr float PShift = 5.f;     // weights are carried times 2^5: keeps small tiles out of the fp16 subnormals
constexpr float PScale = 32.f;    // 2^PShift
enum Mode : int { ModeF16 = 0, ModeI8 = 1, ModeQ4 = 2 };

struct QuadPlan {   // tile visiting order of one CTA (four query blocks q0..q0+3), all warp-uniform integers
  int q0, nb, nF, lo8, n8, lo4, n4, w8, w4;
  __device__ void build(int quad, int rows, int w8_, int w4_) {
    w8 = w8_; w4 = w4_;
    q0 = 4 * quad; nb = min(4, rows - q0);
    nF = 1 + nb - (q0 == 0 ? 1 : 0);   // the sink tile (all blocks; it is also block 0's diagonal tile), then one diagonal tile per block
    // prefill_sm80.cu:281-283 per block, then the union of the contiguous ranges
    int lo = 1 << 30, hi = 0, lq = 1 << 30, hq = 0;
    for (int j = 0; j < nb; ++j) {
      const int qb = q0 + j, l8 = max(1, qb - w8 + 1), c8 = max(0, qb - l8);
      const int l4 = max(1, qb - w4 + 1), c4 = max(0, qb - w8 - l4 + 1);
      if (c8 > 0) { lo = min(lo, l8); hi = max(hi, l8 + c8); }
      if (c4 > 0) { lq = min(lq, l4); hq = max(hq, l4 + c4); }
    }
    lo8 = lo; n8 = max(0, hi - lo); lo4 = lq; n4 = max(0, hq - lq);
  }
  __device__ int steps() const { return nF + n8 + n4; }
  __device__ void get(int i, int& tile, int& mode, int& mask) const {
    if (i < nF) {
      mode = ModeF16;
      if (i == 0) { tile = 0; mask = (1 << nb) - 1; return; }
      const int j = i - 1 + (q0 == 0 ? 1 : 0);
      tile = q0 + j; mask = 1 << j;
      return;
    }
    mask = 0;
    if (i < nF + n8) {
      tile = lo8 + (i - nF); mode = ModeI8;
      for (int j = 0; j < nb; ++j) {
        const int qb = q0 + j;
        if (tile >= max(1, qb - w8 + 1) && tile <= qb - 1) mask |= 1 << j;
      }
    } else {
      tile = lo4 + (i - nF - n8); mode = ModeQ4;
      for (int j = 0; j < nb; ++j) {
        const int qb = q0 + j;
        if (tile >= max(1, qb - w4 + 1) && tile <= qb - w8) mask |= 1 << j;
      }
    }
  }
};

template <typename Out> __device__ __forceinline__ Out to_out(float x);
template <> __device__ __forceinline__ __nv_bfloat16 to_out<__nv_bfloat16>(float x) { return __float2bfloat16(x); }
template <> __device__ __forceinline__ __half to_out<__half>(float x) { return __float2half(x); }

#include "prefill_kernel.cuh"

// ---- integer QK^T accumulators of chosen (Q unit, pair, tile) through the production operand path ---
// grid = requests, 128 threads.  req = {qunit, pair, tile, four_bit}; writes int32 [req][128][64].
__global__ void __launch_bounds__(ProbeThreads) qk_accum_kernel(const __grid_constant__ CUtensorMap map_q8,
    const __grid_constant__ CUtensorMap map_q4, const int4* req, const uint8_t* k8, const uint8_t* k4x, int32_t* acc, int heads_q,
    int heads_kv, int tokens, int* err) {
  extern __shared__ uint8_t raw_smem[];
  __shared__ __align__(8) uint64_t bar_ld, bar_s;
  __shared__ uint32_t tmem_slot;
  uint8_t* smem = raw_smem + ((1024u - (smem_u32(raw_smem) & 1023u)) & 1023u);
  const int tid = threadIdx.x, warp = tid / 32;
  const int4 r = req[blockIdx.x];
  const int tiles = (tokens + BN - 1) / BN, g = heads_q / heads_kv;
  const int64_t kvunit = (int64_t)(r.x / heads_q) * heads_kv + (r.x % heads_q) / g;
  if (tid == 0) { mbar_init(&bar_ld, 1); mbar_init(&bar_s, 1); mbar_fence_init(); }
  if (warp == 0) { tmem_alloc(&tmem_slot, 64); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_slot;
  bool ok = true;
  if (tid == 0) {
    mbar_expect_tx(&bar_ld, 16384u + K8Bytes);
    tma_load_3d(smem, r.w ? &map_q4 : &map_q8, 0, r.y * 2 * BM, r.x, &bar_ld);
    bulk_g2s(smem + 16384, (r.w ? k4x : k8) + (kvunit * tiles + r.z) * K8Bytes, K8Bytes, &bar_ld);
    ok = mbar_wait(&bar_ld, 0);
    if (ok) {
      tc_fence_after();
      const uint32_t qa_ = smem_u32(smem), ka_ = smem_u32(smem + 16384);
#pragma unroll
      for (int kk = 0; kk < 4; ++kk)
        umma_i8(tmem, smem_desc(qa_ + kk * 32, 0, 1024, Layout128B), smem_desc(ka_ + kk * 256, 128, 1024, LayoutNone), IdescQK, kk > 0);
      tc_commit(&bar_s);
    }
  }
  __syncwarp();
  ok = mbar_wait(&bar_s, 0);
  ok = __syncthreads_and(ok);
  if (ok) {
    tc_fence_after();
    int32_t* dst = acc + ((int64_t)blockIdx.x * 128 + tid) * 64;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      uint32_t a[16];
      tmem_ld16(tmem + ((uint32_t)(warp * 32) << 16) + c * 16, a);
      tmem_ld_wait();
#pragma unroll
      for (int j = 0; j < 16; ++j) dst[c * 16 + j] = (int)a[j];
    }
  } else if (tid == 0) {
    atomicExch(err, ErrBarrierTimeout);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, 64);
}

// ---- host side ----------------------------------------------------------------------------------
using EncodeTiled = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                 const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                 CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiled encode_fn() {
  static EncodeTiled fn = nullptr;
  if (fn == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiled>(p);
  }
  return fn;
}

// int8 rows [units][tokens][128]: box = 128 rows x 128 bytes of one unit, 128-byte swizzle, rows past
// `tokens` are filled with zeros by the copy engine.
static int make_q_map(CUtensorMap* map, const void* base, int tokens, int units) {
  EncodeTiled enc = encode_fn();
  TRI_CHECK(enc != nullptr, "cuTensorMapEncodeTiled is not available from this driver");
  const cuuint64_t dims[3] = {(cuuint64_t)D, (cuuint64_t)tokens, (cuuint64_t)units};
  const cuuint64_t strides[2] = {(cuuint64_t)D, (cuuint64_t)tokens * D};
  const cuuint32_t box[3] = {(cuuint32_t)D, 128u, 1u}, estr[3] = {1u, 1u, 1u};
  const CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void*>(base), dims, strides, box, estr,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  TRI_CHECK(r == CUDA_SUCCESS, "cuTensorMapEncodeTiled failed for the Q operand");
  return TRI_OK;
}

// bf16 rows of a caller's [B,H,T,128] tensor with element strides: box = `rows` tokens x 64 features (128 bytes) of one
// head, 128-byte swizzle, tokens past `tokens` filled with zeros.  Coordinates (feature, token, head, sequence).
static int make_raw_map(CUtensorMap* map, const void* base, int tokens, int heads, int batch, int64_t sb, int64_t sh, int64_t st,
                        unsigned rows) {
  EncodeTiled enc = encode_fn();
  TRI_CHECK(enc != nullptr, "cuTensorMapEncodeTiled is not available from this driver");
  const cuuint64_t dims[4] = {(cuuint64_t)D, (cuuint64_t)tokens, (cuuint64_t)heads, (cuuint64_t)batch};
  const cuuint64_t strides[3] = {(cuuint64_t)st * 2, (cuuint64_t)sh * 2, (cuuint64_t)sb * 2};
  const cuuint32_t box[4] = {64u, rows, 1u, 1u}, estr[4] = {1u, 1u, 1u, 1u};
  const CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides, box, estr,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  TRI_CHECK(r == CUDA_SUCCESS, "cuTensorMapEncodeTiled failed for the raw Q / K rows of un-quantised heads");
  return TRI_OK;
}

template <typename K> static int allow_smem(K kernel, int bytes) {
  TRI_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes), "smem attribute");
  return TRI_OK;
}

}  // namespace tri

using namespace tri;

// Shared by tri_attention and tri_attention_sweep: `configs` band tables evaluated in one launch (grid.y), query blocks
// from `first_block` on (the grid covers the quads that contain them), outputs `out_stride_c` elements apart.
static int launch_attention(const int32_t* bands, int configs, int first_block, const void* v16, const void* v8h, const float* vstat,
    const void* q8, const void* k8, const float* qa8, const float* ka8, const void* q4x, const void* k4x, const float* qa4,
    const float* ka4, void* out, int out_is_half, int64_t out_stride_c, int64_t out_stride_b, int64_t out_stride_h,
    int64_t out_stride_t, int batch, int heads_q, int heads_kv, int tokens, double scale, const void* q_raw, int64_t q_stride_b,
    int64_t q_stride_h, int64_t q_stride_t, const void* k_raw, int64_t k_stride_b, int64_t k_stride_h, int64_t k_stride_t,
    int* device_error, void* stream) {
  TRI_CHECK(bands && v16 && vstat && q8 && k8 && qa8 && ka8 && out && device_error, "attention: null buffers");
  TRI_CHECK((q_raw == nullptr) == (k_raw == nullptr), "attention: raw Q and K rows of un-quantised heads (both or none)");
  TRI_CHECK(q_raw == nullptr || (aligned16(q_raw) && aligned16(k_raw) && q_stride_b % 8 == 0 && q_stride_h % 8 == 0 &&
                                 q_stride_t % 8 == 0 && k_stride_b % 8 == 0 && k_stride_h % 8 == 0 && k_stride_t % 8 == 0 &&
                                 q_stride_t >= D && k_stride_t >= D),
            "attention: raw BF16 Q/K [B,H,T,128] rows must be 16-byte aligned");
  TRI_CHECK(batch > 0 && heads_q > 0 && heads_kv > 0 && heads_q % heads_kv == 0 && tokens > 0, "attention: bad geometry");
  TRI_CHECK((tokens + BN - 1) / BN <= MaxTiles, "at most 131072 tokens");
  const bool int4 = q4x != nullptr;
  TRI_CHECK(int4 == (k4x != nullptr) && int4 == (qa4 != nullptr) && int4 == (ka4 != nullptr), "INT4 Q/K operands (all or none)");
  TRI_CHECK(aligned16(out) && out_stride_t % 8 == 0 && out_stride_h % 8 == 0 && out_stride_b % 8 == 0 && out_stride_c % 8 == 0,
            "output [B,Hq,T,128] aligned");
  TRI_CHECK(aligned16(q8) && aligned16(q4x) && aligned16(k8) && aligned16(k4x) && aligned16(v16) && aligned16(v8h),
            "attention: operands must be 16-byte aligned");
  const int units = batch * heads_q, rows = (tokens + BM - 1) / BM, quads = (rows + 3) / 4;
  TRI_CHECK(configs >= 1 && configs <= 65535 && first_block >= 0 && first_block < rows, "attention: configurations / first query block");
  static TriPerDevice configured;
  const int device = configured.pending();
  TRI_CHECK(device != -2, "attention: no current CUDA device");
  if (device >= 0) {
    if (allow_smem(prefill_kernel<__nv_bfloat16, false>, PrefillShared) != TRI_OK) return TRI_ERR_CUDA;
    if (allow_smem(prefill_kernel<__half, false>, PrefillShared) != TRI_OK) return TRI_ERR_CUDA;
    if (allow_smem(prefill_kernel<__nv_bfloat16, true>, PrefillShared) != TRI_OK) return TRI_ERR_CUDA;
    if (allow_smem(prefill_kernel<__half, true>, PrefillShared) != TRI_OK) return TRI_ERR_CUDA;
    configured.mark(device);
  }
  CUtensorMap map8, map4, mapq, mapk;
  if (make_q_map(&map8, q8, tokens, units) != TRI_OK) return TRI_ERR_CUDA;
  if (make_q_map(&map4, int4 ? q4x : q8, tokens, units) != TRI_OK) return TRI_ERR_CUDA;
  const int has_raw = q_raw != nullptr ? 1 : 0;
  if (has_raw) {
    if (make_raw_map(&mapq, q_raw, tokens, heads_q, batch, q_stride_b, q_stride_h, q_stride_t, 128u) != TRI_OK) return TRI_ERR_CUDA;
    if (make_raw_map(&mapk, k_raw, tokens, heads_kv, batch, k_stride_b, k_stride_h, k_stride_t, 64u) != TRI_OK) return TRI_ERR_CUDA;
  } else {
    mapq = map8; mapk = map8;   // never dereferenced: heads with w8 < 1 are skipped when no raw rows are given
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const float sm_log2 = (float)(scale * 1.4426950408889634);
  // CTA x = (quads - 1 - quad) * units + unit, heaviest quads first: the first (quads - first_quad) * units CTAs are
  // exactly the quads that hold query blocks >= first_block
  const dim3 grid((unsigned)((int64_t)(quads - first_block / 4) * units), (unsigned)configs);
#define TRI_LAUNCH(T, R)                                                                                                   \
  prefill_kernel<T, R><<<grid, PrefillThreads, PrefillShared, s>>>(map8, map4, mapq, mapk, has_raw, bands,                \
      static_cast<const uint8_t*>(k8),                                                                                     \
      static_cast<const uint8_t*>(k4x), ka8, ka4, static_cast<const uint8_t*>(v16), static_cast<const uint8_t*>(v8h), qa8, \
      qa4, vstat, static_cast<T*>(out), out_stride_b, out_stride_h, out_stride_t, out_stride_c, heads_q, heads_kv, tokens, \
      units, sm_log2, device_error)
  // quantised heads, then (if the map has any) the un-quantised ones: the same kernel, instantiated for each kind
  if (out_is_half) TRI_LAUNCH(__half, false); else TRI_LAUNCH(__nv_bfloat16, false);
  if (has_raw) {
    if (out_is_half) TRI_LAUNCH(__half, true); else TRI_LAUNCH(__nv_bfloat16, true);
  }
#undef TRI_LAUNCH
  return tri_launch_status("attention");
}

extern "C" int tri_attention(const int32_t* bands, const void* v16, const void* v8h, const float* vstat, const void* q8,
    const void* k8, const float* qa8, const float* ka8, const void* q4x, const void* k4x, const float* qa4, const float* ka4,
    void* out, int out_is_half, int64_t out_stride_b, int64_t out_stride_h, int64_t out_stride_t, int batch, int heads_q,
    int heads_kv, int tokens, double scale, const void* q_raw, int64_t q_stride_b, int64_t q_stride_h, int64_t q_stride_t,
    const void* k_raw, int64_t k_stride_b, int64_t k_stride_h, int64_t k_stride_t, int* device_error, void* stream) {
  return launch_attention(bands, 1, 0, v16, v8h, vstat, q8, k8, qa8, ka8, q4x, k4x, qa4, ka4, out, out_is_half, 0, out_stride_b,
                          out_stride_h, out_stride_t, batch, heads_q, heads_kv, tokens, scale, q_raw, q_stride_b, q_stride_h,
                          q_stride_t, k_raw, k_stride_b, k_stride_h, k_stride_t, device_error, stream);
}

extern "C" int tri_attention_sweep(const int32_t* bands, int configs, int first_block, const void* v16, const void* v8h,
    const float* vstat, const void* q8, const void* k8, const float* qa8, const float* ka8, const void* q4x, const void* k4x,
    const float* qa4, const float* ka4, void* out, int out_is_half, int64_t out_stride_c, int64_t out_stride_b,
    int64_t out_stride_h, int64_t out_stride_t, int batch, int heads_q, int heads_kv, int tokens, double scale,
    int* device_error, void* stream) {
  return launch_attention(bands, configs, first_block, v16, v8h, vstat, q8, k8, qa8, ka8, q4x, k4x, qa4, ka4, out, out_is_half,
                          out_stride_c, out_stride_b, out_stride_h, out_stride_t, batch, heads_q, heads_kv, tokens, scale, nullptr,
                          0, 0, 0, nullptr, 0, 0, 0, device_error, stream);
}

extern "C" int tri_qk_accumulators(const int32_t* requests, int num_requests, const void* q8, const void* q4x, const void* k8,
    const void* k4x, int32_t* acc, int batch, int heads_q, int heads_kv, int tokens, int* device_error, void* stream) {
  TRI_CHECK(requests && q8 && k8 && acc && device_error && num_requests > 0, "qk_accumulators: null buffers");
  TRI_CHECK(batch > 0 && heads_q > 0 && heads_kv > 0 && heads_q % heads_kv == 0 && tokens > 0, "qk_accumulators: bad geometry");
  static TriPerDevice configured;
  const int device = configured.pending();
  TRI_CHECK(device != -2, "qk_accumulators: no current CUDA device");
  if (device >= 0) {
    if (allow_smem(qk_accum_kernel, 16384 + K8Bytes + 1024) != TRI_OK) return TRI_ERR_CUDA;
    configured.mark(device);
  }
  const int units = batch * heads_q;
  CUtensorMap map8, map4;
  if (make_q_map(&map8, q8, tokens, units) != TRI_OK) return TRI_ERR_CUDA;
  if (make_q_map(&map4, q4x ? q4x : q8, tokens, units) != TRI_OK) return TRI_ERR_CUDA;
  qk_accum_kernel<<<num_requests, ProbeThreads, 16384 + K8Bytes + 1024, static_cast<cudaStream_t>(stream)>>>(map8, map4,
      reinterpret_cast<const int4*>(requests), static_cast<const uint8_t*>(k8), static_cast<const uint8_t*>(k4x ? k4x : k8), acc,
      heads_q, heads_kv, tokens, device_error);
  return tri_launch_status("qk_accumulators");
}
