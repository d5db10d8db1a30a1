// Split-KV decode over the mixed-width KV cache, sm_100a: host launchers, the merge kernel and the
// cache-store (gather + re-layout) kernels.  The streaming kernel itself is in decode_kernel.cuh.
//
// Replaces (paths inside the reference project)
//   triattention/kernels/cuda/common_device.cuh:178-371  decode_tile, decode_kernel
//   triattention/kernels/cuda/common_device.cuh:373-469  decode_merge_kernel
//   triattention/kernels/cuda/common_host.cuh:47-94      decode, decode_occupancy
//   triattention/kernels/decode.py:46-61                 the index_select gathers of DecodeCache.store
// with a batch dimension, a cost-balanced static partition of the tile sequence over persistent CTAs
// instead of a fixed tiles-per-split, and an un-quantised BF16 head kind that the reference lacks.
#include "decode_kernel.cuh"
#include "abi_internal.h"

namespace tri {

// grid (heads_q, batch), 256 threads.  common_device.cuh:373-469 with per-unit split ranges.
constexpr int MergeThreads = 256;
__global__ void __launch_bounds__(MergeThreads) decode_merge_kernel(const float* pm, const float* pl, const float* po,
    const int2* unit_slots, const float* vstat, const float* kstat, const __nv_bfloat16* q, int64_t qsb, int64_t qsh,
    __nv_bfloat16* ktail, __nv_bfloat16* vtail, int64_t tsu, int64_t tst, const __nv_bfloat16* kcur,
    const __nv_bfloat16* vcur, int64_t csb, int64_t csh, const int64_t* step, __nv_bfloat16* out, int64_t osb, int64_t osh,
    int heads_q, int heads_kv, int max_tail, float sm_log2) {
  constexpr int W = MergeThreads / 32;
  __shared__ float ts[1024];
  __shared__ __align__(16) float ew[1024];
  __shared__ float wmax[W], wl[W];
  __shared__ __align__(16) float wo[W][D];
  const int hq = blockIdx.x, b = blockIdx.y, g = heads_q / heads_kv, kh = hq / g, r = hq % g;
  const int unit = b * heads_kv + kh, tid = threadIdx.x, lane = tid % 32, warp = tid / 32;
  grid_launch_dependents();   // the next step's split pass may set up its barriers behind this kernel
  grid_dependency_wait();     // the split pass has written all partials
  const int prior = min((int)*step, max_tail - 1), tail = prior + 1;
  const float* mean = vstat + (int64_t)unit * StatFloats;
  const float* scale = mean + D;
  const __nv_bfloat16* kc = kcur + b * csb + kh * csh;
  const __nv_bfloat16* vc = vcur + b * csb + kh * csh;
  __nv_bfloat16* kt = ktail + unit * tsu;
  __nv_bfloat16* vt = vtail + unit * tsu;
  if (r == 0 && tid < D) {
    kt[prior * tst + tid] = kc[tid];
    vt[prior * tst + tid] = vc[tid];
  }
  const __nv_bfloat16* qrow = q + b * qsb + hq * qsh;
  float qv[4], kmean[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) { qv[i] = __bfloat162float(qrow[lane * 4 + i]); kmean[i] = kstat[(int64_t)unit * StatFloats + lane * 4 + i]; }
  for (int t = warp; t < tail; t += W) {
    const __nv_bfloat16* kv = t < prior ? kt + t * tst : kc;
    float part = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) part = fmaf(qv[i], __bfloat162float(kv[lane * 4 + i]) - kmean[i], part);
#pragma unroll
    for (int o = 16; o; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
    if (lane == 0) ts[t] = part * sm_log2;
  }
  __syncthreads();
  const int2 sl = unit_slots[unit];
  const int sbeg = sl.x, splits = sl.y;
  float m = -FLT_MAX;
  for (int s = tid; s < splits; s += MergeThreads) m = fmaxf(m, pm[(int64_t)(sbeg + s) * MaxGroup + r]);
  for (int t = tid; t < tail; t += MergeThreads) m = fmaxf(m, ts[t]);
#pragma unroll
  for (int o = 16; o; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  if (lane == 0) wmax[warp] = m;
  __syncthreads();
  m = wmax[0];
#pragma unroll
  for (int w = 1; w < W; ++w) m = fmaxf(m, wmax[w]);
  for (int t = tid; t < tail; t += MergeThreads) ew[t] = exp2f(ts[t] - m);
  float l = 0.f, o[4] = {0.f, 0.f, 0.f, 0.f};
  for (int s = warp; s < splits; s += W) {
    const int64_t idx = (int64_t)(sbeg + s) * MaxGroup + r;
    const float w = exp2f(pm[idx] - m);
    l = fmaf(pl[idx], w, l);
    const float4 p = *reinterpret_cast<const float4*>(po + idx * D + lane * 4);
    o[0] = fmaf(p.x, w, o[0]); o[1] = fmaf(p.y, w, o[1]); o[2] = fmaf(p.z, w, o[2]); o[3] = fmaf(p.w, w, o[3]);
  }
  if (lane == 0) wl[warp] = l;
  *reinterpret_cast<float4*>(&wo[warp][lane * 4]) = make_float4(o[0], o[1], o[2], o[3]);
  __syncthreads();
  if (tid >= D) return;
  float total = 0.f, acc = 0.f;
#pragma unroll
  for (int w = 0; w < W; ++w) { total += wl[w]; acc += wo[w][tid]; }
  acc = acc * scale[tid] + total * mean[tid];
  for (int t = 0; t < prior; ++t) {
    const float e = ew[t];
    total += e;
    acc = fmaf(e, __bfloat162float(vt[(int64_t)t * tst + tid]), acc);
  }
  total += ew[prior];
  acc = fmaf(ew[prior], __bfloat162float(vc[tid]), acc);
  out[b * osb + hq * osh + tid] = __float2bfloat16(acc / total);
}


// ---- cache store: gather kept tiles of the prefill operands into the per-unit streams ------------
// grid (max kept tiles, units), 256 threads.  K8 / V8 / V4 blobs are re-ordered from the prefill
// operand layout (tcgen05 core matrices, csrc/common.cuh) into the decode layout (decode_kernel.cuh):
// the same codes, permuted in 16-byte units (K8) or 32-bit words (V8, V4).  K4 blobs are already
// written in the decode layout.
__global__ void __launch_bounds__(256) cache_store_kernel(uint8_t* pool, const int64_t* unit_base, const int32_t* unit_tab,
    const int32_t* unit_count, const int32_t* unit_flags, const int2* tmeta, const uint8_t* k8, const uint8_t* k4,
    const float* ka, const float* ka4, const uint8_t* v8, const uint8_t* v4, int tiles) {
  const int i = blockIdx.x, unit = blockIdx.y, tid = threadIdx.x;
  if (i >= unit_count[unit] || (unit_flags[unit] & 1)) return;
  const int2 mt = tmeta[unit_tab[unit] + i];
  const uint32_t info = (uint32_t)mt.y;
  const int64_t ht = (int64_t)unit * tiles + (info & InfoTileMask);
  uint8_t* dst = pool + unit_base[unit] + (int64_t)mt.x * 16;
  const bool is_k4 = info & InfoK4, is_v4 = info & InfoV4;
  if (is_k4) {
    const uint4* src = reinterpret_cast<const uint4*>(k4 + ht * K4Bytes);
    for (int d = tid; d < K4Bytes / 16; d += 256) reinterpret_cast<uint4*>(dst)[d] = src[d];
  } else {
    const uint4* src = reinterpret_cast<const uint4*>(k8 + ht * K8Bytes);
    for (int d = tid; d < K8Bytes / 16; d += 256) {
      const int blk = d / 64, h = (d % 64) / 32, key = (d % 32) / 4, sub = d % 4;
      reinterpret_cast<uint4*>(dst)[d] = src[blk * 64 + (2 * sub + h) * 8 + key];
    }
  }
  uint8_t* vd = dst + (is_k4 ? K4Bytes : K8Bytes);
  if (is_v4) {
    const uint32_t* src = reinterpret_cast<const uint32_t*>(v4 + ht * V4Bytes);
    for (int d = tid; d < V4Bytes / 8; d += 256) {      // one 8-byte run = (channel, sub): words kc = 0, 1
      const int cb = d / 32, ch = (d % 32) / 4, sub = d % 4;
      reinterpret_cast<uint2*>(vd)[d] = make_uint2(src[cb * 64 + ch * 4 + sub], src[cb * 64 + 32 + ch * 4 + sub]);
    }
  } else {
    const uint32_t* src = reinterpret_cast<const uint32_t*>(v8 + ht * V8Bytes);
    for (int d = tid; d < V8Bytes / 16; d += 256) {     // one 16-byte run = (channel, sub): words of key groups 0..3
      const int cb = d / 32, ch = (d % 32) / 4, sub = d % 4;
      const uint32_t* s = src + cb * 128 + ch * 4 + sub;
      reinterpret_cast<uint4*>(vd)[d] = make_uint4(s[0], s[32], s[64], s[96]);
    }
  }
  if (tid == 0)
    *reinterpret_cast<uint4*>(vd + (is_v4 ? V4Bytes : V8Bytes)) = *reinterpret_cast<const uint4*>((is_k4 ? ka4 : ka) + ht * 4);
}

// grid (32-key chunks, listed BF16 units), 256 threads: K/V bf16 [B,Hkv,T,128] -> decode-layout chunks.
__global__ void __launch_bounds__(256) cache_store_bf16_kernel(uint8_t* pool, const int64_t* unit_base, const int32_t* units,
    const __nv_bfloat16* k, const __nv_bfloat16* v, int tokens, int heads, int64_t ksb, int64_t ksh, int64_t kst, int64_t vsb,
    int64_t vsh, int64_t vst, int chunk_begin) {
  const int unit = units[blockIdx.y];
  const __nv_bfloat16* kb = k + (unit / heads) * ksb + (unit % heads) * ksh;
  const __nv_bfloat16* vb = v + (unit / heads) * vsb + (unit % heads) * vsh;
  uint8_t* dst = pool + unit_base[unit] + (int64_t)blockIdx.x * Bf16ChunkBytes;   // the stream holds chunks begin, begin+1, ...
  const int key0 = (chunk_begin + blockIdx.x) * Bf16ChunkKeys;
  for (int d = threadIdx.x; d < 512; d += 256) {      // K: 16-byte runs [key/8][u][key%8][sub] = features 32sub+8u..+7
    const int nb = d / 128, u = (d % 128) / 32, key = key0 + nb * 8 + (d % 32) / 4, sub = d % 4;
    reinterpret_cast<uint4*>(dst)[d] = key < tokens ? *reinterpret_cast<const uint4*>(kb + (int64_t)key * kst + sub * 32 + u * 8)
                                                    : make_uint4(0, 0, 0, 0);
  }
  uint32_t* vd = reinterpret_cast<uint32_t*>(dst + 8192);
  for (int w = threadIdx.x; w < 2048; w += 256) {     // V words [ch/8][ch%8][sub][2ks+h] = keys 16ks+8h+2sub+{0,1}
    const int cb = w / 128, ch = cb * 8 + (w % 128) / 16, sub = (w % 16) / 4, ks = (w % 4) / 2, h = w % 2;
    const int key = key0 + ks * 16 + h * 8 + sub * 2;
    const uint32_t lo = key < tokens ? __bfloat16_as_ushort(vb[(int64_t)key * vst + ch]) : 0u;
    const uint32_t hi = key + 1 < tokens ? __bfloat16_as_ushort(vb[(int64_t)(key + 1) * vst + ch]) : 0u;
    vd[w] = lo | (hi << 16);
  }
}

static int configure_decode() {
  static int done = 0;   // per process; the attribute is per function
  if (!done) {
    TRI_CUDA(cudaFuncSetAttribute(decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, DecodeShared), "decode");
    done = 1;
  }
  return TRI_OK;
}

}  // namespace tri

using namespace tri;

extern "C" int tri_decode_occupancy(void) {
  if (configure_decode() != TRI_OK) return TRI_ERR_CUDA;
  int blocks = 0;
  TRI_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&blocks, decode_kernel, DecodeThreads, DecodeShared), "decode_occupancy");
  return blocks;
}

extern "C" int tri_decode(const void* q, int64_t q_stride_b, int64_t q_stride_h, const void* pool, const int64_t* unit_base,
    const int32_t* unit_tab, const int32_t* unit_flags, const int32_t* tmeta, const int32_t* segments, const int32_t* cta_segments,
    int num_ctas, const int32_t* unit_slots, const float* kstat, const float* vstat, void* tail_k, void* tail_v,
    int64_t tail_stride_u, int64_t tail_stride_t, const void* kcur, const void* vcur, int64_t cur_stride_b,
    int64_t cur_stride_h, const int64_t* step, void* out, int64_t out_stride_b, int64_t out_stride_h, float* pm, float* pl,
    float* po, int32_t* unit_done, int batch, int heads_q, int heads_kv, int prompt, int max_tail, double scale, int phases,
    int* device_error, void* stream) {
  TRI_CHECK(q && pool && unit_base && unit_tab && unit_flags && tmeta && segments && cta_segments && unit_slots && kstat &&
            vstat && tail_k && tail_v && kcur && vcur && step && out && pm && pl && po && device_error, "decode: null buffers");
  TRI_CHECK(batch > 0 && heads_q > 0 && heads_kv > 0 && heads_q % heads_kv == 0 && heads_q / heads_kv <= MaxGroup &&
            max_tail >= 1 && max_tail <= 1024 && prompt > 0 && num_ctas >= 0, "decode geometry/buffers");
  TRI_CHECK(aligned16(pool) && aligned16(po) && (reinterpret_cast<uintptr_t>(q) & 7u) == 0 && q_stride_b % 4 == 0 &&
            q_stride_h % 4 == 0, "decode: alignment");
  if (configure_decode() != TRI_OK) return TRI_ERR_CUDA;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const float sm_log2 = (float)(scale * 1.4426950408889634);
  const auto* qp = static_cast<const __nv_bfloat16*>(q);
  // One launch when both phases are wanted and the caller provides the per-unit completion counters: the CTA
  // that finishes a unit's last segment merges it.  Otherwise the split pass and the merge are two launches.
  const bool fused = phases == 3 && unit_done != nullptr && num_ctas > 0;
  MergeArgs margs{};
  if (fused)
    margs = MergeArgs{reinterpret_cast<const int2*>(unit_slots), unit_done, vstat, kstat, static_cast<__nv_bfloat16*>(tail_k),
                      static_cast<__nv_bfloat16*>(tail_v), tail_stride_u, tail_stride_t, static_cast<const __nv_bfloat16*>(kcur),
                      static_cast<const __nv_bfloat16*>(vcur), cur_stride_b, cur_stride_h, step, static_cast<__nv_bfloat16*>(out),
                      out_stride_b, out_stride_h, max_tail};
  if (num_ctas > 0 && (phases & 1))
    launch_chained(decode_kernel, dim3(num_ctas), dim3(DecodeThreads), DecodeShared, s, qp, q_stride_b, q_stride_h,
        static_cast<const uint8_t*>(pool), unit_base, unit_tab, unit_flags, reinterpret_cast<const int2*>(tmeta),
        reinterpret_cast<const int4*>(segments), cta_segments, pm, pl, po, heads_q, heads_kv, prompt, sm_log2,
        (phases & 4) ? 1 : 0, margs, device_error);
  if ((phases & 2) && !fused)
    launch_chained(decode_merge_kernel, dim3(heads_q, batch), dim3(MergeThreads), 0, s, pm, pl, po,
        reinterpret_cast<const int2*>(unit_slots), vstat, kstat, qp, q_stride_b, q_stride_h, static_cast<__nv_bfloat16*>(tail_k), static_cast<__nv_bfloat16*>(tail_v),
        tail_stride_u, tail_stride_t, static_cast<const __nv_bfloat16*>(kcur), static_cast<const __nv_bfloat16*>(vcur),
        cur_stride_b, cur_stride_h, step, static_cast<__nv_bfloat16*>(out), out_stride_b, out_stride_h, heads_q, heads_kv,
        max_tail, sm_log2);
  return tri_launch_status("decode");
}

extern "C" int tri_cache_store(void* pool, const int64_t* unit_base, const int32_t* unit_tab, const int32_t* unit_count,
    const int32_t* unit_flags, const int32_t* tmeta, int units, int max_count, const void* k8, const void* k4, const float* ka,
    const float* ka4, const void* v8, const void* v4, int tiles, void* stream) {
  TRI_CHECK(pool && unit_base && unit_tab && unit_count && unit_flags && tmeta && k8 && ka && v8, "cache_store: null buffers");
  TRI_CHECK(units > 0 && max_count > 0 && tiles > 0 && aligned16(pool) && aligned16(k8) && aligned16(k4) && aligned16(v8) &&
            aligned16(v4) && aligned16(ka) && aligned16(ka4), "cache_store: geometry/alignment");
  cache_store_kernel<<<dim3(max_count, units), 256, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<uint8_t*>(pool),
      unit_base, unit_tab, unit_count, unit_flags, reinterpret_cast<const int2*>(tmeta), static_cast<const uint8_t*>(k8),
      static_cast<const uint8_t*>(k4), ka, ka4, static_cast<const uint8_t*>(v8), static_cast<const uint8_t*>(v4), tiles);
  return tri_launch_status("cache_store");
}

extern "C" int tri_cache_store_bf16(void* pool, const int64_t* unit_base, const int32_t* units, int num_units, const void* k,
    const void* v, int tokens, int heads_kv, int64_t k_stride_b, int64_t k_stride_h, int64_t k_stride_t, int64_t v_stride_b,
    int64_t v_stride_h, int64_t v_stride_t, int chunk_begin, int chunk_count, void* stream) {
  TRI_CHECK(pool && unit_base && units && k && v && num_units > 0 && tokens > 0 && heads_kv > 0, "cache_store_bf16: arguments");
  TRI_CHECK(k_stride_t % 8 == 0 && k_stride_h % 8 == 0 && k_stride_b % 8 == 0 && aligned16(k) && aligned16(pool),
            "cache_store_bf16: K rows must be 16-byte aligned");
  const int chunks = (tokens + Bf16ChunkKeys - 1) / Bf16ChunkKeys;
  TRI_CHECK(chunk_begin >= 0 && chunk_count > 0 && chunk_begin + chunk_count <= chunks, "cache_store_bf16: chunk range");
  cache_store_bf16_kernel<<<dim3(chunk_count, num_units), 256, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<uint8_t*>(pool),
      unit_base, units, static_cast<const __nv_bfloat16*>(k), static_cast<const __nv_bfloat16*>(v), tokens, heads_kv,
      k_stride_b, k_stride_h, k_stride_t, v_stride_b, v_stride_h, v_stride_t, chunk_begin);
  return tri_launch_status("cache_store_bf16");
}

// ---- fold: one (m, l, o) per unit and Q head from the unit's segment partials ---------------------
// Used when a unit's tile range is split across GPUs: every rank folds its local segments, the
// folded triples (1,040 B per Q head) are all-gathered, and the merge kernel then sees one "segment" per
// rank.  Same arithmetic as the first half of decode_merge_kernel; no V de-normalisation, no tail.
namespace tri {
__global__ void __launch_bounds__(D) decode_fold_kernel(const float* pm, const float* pl, const float* po,
    const int2* unit_slots, float* fm, float* fl, float* fo, int group) {
  const int unit = blockIdx.x, ch = threadIdx.x;
  const int2 sl = unit_slots[unit];
  for (int r = 0; r < group; ++r) {
    float big = -FLT_MAX;
    for (int s = 0; s < sl.y; ++s) big = fmaxf(big, pm[(int64_t)(sl.x + s) * MaxGroup + r]);
    float o = 0.f, l = 0.f;
    for (int s = 0; s < sl.y; ++s) {
      const int64_t idx = (int64_t)(sl.x + s) * MaxGroup + r;
      const float w = exp2f(pm[idx] - big);
      o = fmaf(po[idx * D + ch], w, o);
      l = fmaf(pl[idx], w, l);
    }
    const int64_t dst = (int64_t)unit * MaxGroup + r;
    fo[dst * D + ch] = o;
    if (ch == 0) { fm[dst] = big; fl[dst] = l; }
  }
}
}  // namespace tri

extern "C" int tri_decode_fold(const float* pm, const float* pl, const float* po, const int32_t* unit_slots, float* fm,
    float* fl, float* fo, int units, int group, void* stream) {
  TRI_CHECK(pm && pl && po && unit_slots && fm && fl && fo, "decode_fold: null buffers");
  TRI_CHECK(units > 0 && group >= 1 && group <= MaxGroup, "decode_fold: geometry");
  decode_fold_kernel<<<units, D, 0, static_cast<cudaStream_t>(stream)>>>(pm, pl, po, reinterpret_cast<const int2*>(unit_slots),
      fm, fl, fo, group);
  return tri_launch_status("decode_fold");
}

// ---- decode step for callers that cannot allocate device memory -----------------------------------
// Some callers of this library own no allocator on the GPU: a serving runtime that has handed every
// byte of HBM to its paged KV pool before the first request arrives, or a host language binding that
// can pass tensors it was given but has no way to ask the driver for more.  tri_decode needs scratch
// for the split-KV partials (pm, pl, po); this variant keeps that scratch inside the library image, in
// a fixed array that every GPU loading the library holds until the process exits.
constexpr int StaticSlots = 1024;                                     // partial slots (segments) per call, at most
constexpr size_t StaticFloats = (size_t)StaticSlots * MaxGroup * (D + 2);
static __device__ __align__(256) float g_static_partials[StaticFloats];   // 4,259,840 bytes per GPU

// Device address of the array, looked up once per device.  In host code the array's name is only a
// handle for the runtime, never an address a kernel may use.
static float* static_partials_for_current_device(void) {
  constexpr int MaxDevices = 64;
  static float* known[MaxDevices] = {};
  int device = -1;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= MaxDevices) return nullptr;
  if (known[device] == nullptr) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_static_partials) != cudaSuccess) return nullptr;
    known[device] = static_cast<float*>(p);
  }
  return known[device];
}

extern "C" int tri_decode_static(const void* q, int64_t q_stride_b, int64_t q_stride_h, const void* pool,
    const int64_t* unit_base, const int32_t* unit_tab, const int32_t* unit_flags, const int32_t* tmeta, const int32_t* segments,
    const int32_t* cta_segments, int num_ctas, int num_slots, const int32_t* unit_slots, const float* kstat, const float* vstat,
    void* tail_k, void* tail_v, int64_t tail_stride_u, int64_t tail_stride_t, const void* kcur, const void* vcur,
    int64_t cur_stride_b, int64_t cur_stride_h, const int64_t* step, void* out, int64_t out_stride_b, int64_t out_stride_h,
    int batch, int heads_q, int heads_kv, int prompt, int max_tail, double scale, int* device_error, void* stream) {
  TRI_CHECK(q && pool && unit_base && unit_tab && unit_flags && tmeta && segments && cta_segments && unit_slots && kstat &&
            vstat && tail_k && tail_v && kcur && vcur && step && out && device_error, "decode_static: null buffers");
  TRI_CHECK(batch > 0 && heads_q > 0 && heads_kv > 0 && heads_q % heads_kv == 0 && heads_q / heads_kv <= MaxGroup &&
            max_tail >= 1 && max_tail <= 1024 && prompt > 0 && num_ctas > 0 && num_slots > 0, "decode geometry/buffers");
  TRI_CHECK(num_slots <= StaticSlots,
            "decode_static: more than 1024 partial slots (segments); use tri_decode with caller-allocated partials");
  TRI_CHECK(aligned16(pool) && (reinterpret_cast<uintptr_t>(q) & 7u) == 0 && q_stride_b % 4 == 0 && q_stride_h % 4 == 0,
            "decode: alignment");
  if (configure_decode() != TRI_OK) return TRI_ERR_CUDA;
  float* scratch = static_partials_for_current_device();
  if (scratch == nullptr) {
    tri_set_error("decode_static: cudaGetSymbolAddress failed for the partials array on the current device");
    return TRI_ERR_CUDA;
  }
  // Nothing in the array has to start at zero: the split pass writes every (slot, Q head) entry that the
  // merge reads, so the previous call's contents are simply overwritten.
  float* pm = scratch;
  float* pl = scratch + (size_t)StaticSlots * MaxGroup;
  float* po = scratch + (size_t)StaticSlots * MaxGroup * 2;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const float sm_log2 = (float)(scale * 1.4426950408889634);
  const auto* qp = static_cast<const __nv_bfloat16*>(q);
  decode_kernel<<<num_ctas, DecodeThreads, DecodeShared, s>>>(qp, q_stride_b, q_stride_h, static_cast<const uint8_t*>(pool),
      unit_base, unit_tab, unit_flags, reinterpret_cast<const int2*>(tmeta), reinterpret_cast<const int4*>(segments),
      cta_segments, pm, pl, po, heads_q, heads_kv, prompt, sm_log2, 0, MergeArgs{}, device_error);
  decode_merge_kernel<<<dim3(heads_q, batch), MergeThreads, 0, s>>>(pm, pl, po, reinterpret_cast<const int2*>(unit_slots), vstat,
      kstat, qp, q_stride_b, q_stride_h, static_cast<__nv_bfloat16*>(tail_k), static_cast<__nv_bfloat16*>(tail_v),
      tail_stride_u, tail_stride_t, static_cast<const __nv_bfloat16*>(kcur), static_cast<const __nv_bfloat16*>(vcur),
      cur_stride_b, cur_stride_h, step, static_cast<__nv_bfloat16*>(out), out_stride_b, out_stride_h, heads_q, heads_kv,
      max_tail, sm_log2);
  return tri_launch_status("decode_static");
}
