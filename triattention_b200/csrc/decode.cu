// Split-KV decode over the mixed-width KV cache, sm_100a.
//
// Replaces (paths inside the reference project)
//   triattention/kernels/cuda/common_device.cuh:178-371  decode_tile, decode_kernel
//   triattention/kernels/cuda/common_device.cuh:373-469  decode_merge_kernel
//   triattention/kernels/cuda/common_host.cuh:47-94      decode, decode_occupancy
//   triattention/kernels/decode.py:46-61                 the index_select gathers of DecodeCache.store
// with a batch dimension, a byte-balanced work list instead of a fixed tiles-per-split, and an
// un-quantised BF16 head kind that the reference does not have.
//
// The kernel is HBM-bound: one 64-key tile is 8-16 KB of codes for at most 8 query rows.  Each work
// item streams a contiguous byte range of one (sequence, KV head) cache stream through a 4-stage
// shared-memory ring filled by TMA bulk copies (cp.async.bulk + mbarrier transaction counts), one
// copy per tile chunk.  The arithmetic per tile is small and runs on warp-level integer MMAs with
// operands read straight from the ring; INT4 codes are widened to int8 (x16) in registers, which
// keeps the integer accumulators exact (they are shifted back).  The float expressions of the
// softmax/P-quantisation are the reference's, so the 8-bit / 4-bit P codes of a tile are the same
// for any split of the tile list.
#include "common.cuh"
#include "abi_internal.h"

namespace tri {

constexpr int DecodeThreads = 128;
constexpr int DecodeStages = 4;
constexpr int StageBytes = 16512;                      // >= 8192 + 8192 + 16, multiple of 128
constexpr int DecodeShared = DecodeStages * StageBytes;
constexpr int Bf16ChunkKeys = 32, Bf16ChunkBytes = 16384;
constexpr int MaxItemTiles = 256;                      // tiles (chunks) per work item; the planner cuts finer than this

// tile_info bits
constexpr uint32_t InfoTileMask = 0xfffu, InfoRowShift = 12, InfoK4 = 1u << 20, InfoV4 = 1u << 21, InfoBf16 = 1u << 22;

__device__ __forceinline__ uint32_t chunk_bytes(uint32_t info) {
  if (info & InfoBf16) return Bf16ChunkBytes;
  return ((info & InfoK4) ? K4Bytes : K8Bytes) + ((info & InfoV4) ? V4Bytes : V8Bytes) + 16;
}

struct RowState {
  float m, denom, corr;
  float out[4][2];
};

// One quantised tile.  Lane (group = lane/4, sub = lane%4) of warp w owns row `group` and keys
// 16w + {2sub, 2sub+1, 8+2sub, 9+2sub} for QK, channels 32w + 8i + 2sub + {0,1} for PV.
template <bool K4, bool V4, typename AfterSync>
__device__ __forceinline__ void quantised_tile(const uint8_t* stage, const uint32_t (&qf)[4][2], float qs, uint32_t* pbuf,
    float* rowmax, RowState& st, int key_begin, int prompt, bool row_on, AfterSync after_sync) {
  const int lane = threadIdx.x % 32, warp = threadIdx.x / 32, group = lane / 4, sub = lane % 4;
  constexpr int KB = K4 ? K4Bytes : K8Bytes, VB = V4 ? V4Bytes : V8Bytes;
  const uint8_t* vb = stage + KB;
  const float* kt = reinterpret_cast<const float*>(stage + KB + VB);
  int c[2][4] = {};
#pragma unroll
  for (int s = 0; s < 4; ++s) {
#pragma unroll
    for (int nb = 0; nb < 2; ++nb) {
      uint32_t b0, b1;
      if constexpr (!K4) {
        const uint32_t* p = reinterpret_cast<const uint32_t*>(stage + (2 * warp + nb) * 1024 + (2 * s) * 128 + group * 16 + sub * 4);
        b0 = p[0]; b1 = p[32];
      } else {
        const uint32_t w = *reinterpret_cast<const uint32_t*>(stage + (2 * warp + nb) * 512 + s * 128 + group * 16 + sub * 4);
        b0 = (w << 4) & 0xf0f0f0f0u; b1 = w & 0xf0f0f0f0u;
      }
      mma_s8(c[nb], qf[s][0], qf[s][1], b0, b1);
    }
  }
  // accumulators in the reference's lane order (common_device.cuh:213-216)
  int acc[4] = {c[0][0], c[0][1], c[1][0], c[1][1]};
  if constexpr (K4) {
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[i] >>= 8;          // both operands were widened by 16
  }
  const float slope[2] = {qs * kt[warp], qs * fmaxf(fmaxf(kt[0], kt[1]), fmaxf(kt[2], kt[3]))};
  float x[4];
  int xbits[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int key = key_begin + warp * 16 + (i >= 2 ? 8 : 0) + sub * 2 + (i % 2);
    xbits[i] = acc[i] + Magic;
    x[i] = (row_on && key < prompt) ? __int_as_float(xbits[i]) : -CUDART_INF_F;
  }
  float mx = fmaxf(fmaxf(x[0], x[1]), fmaxf(x[2], x[3]));
  mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
  mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
  if (sub == 0) rowmax[warp * 8 + group] = mx > -CUDART_INF_F ? slope[0] * __fsub_rn(mx, 12582912.f) : -CUDART_INF_F;
  __syncthreads();
  after_sync();
  const float tile = fmaxf(fmaxf(rowmax[group], rowmax[8 + group]), fmaxf(rowmax[16 + group], rowmax[24 + group]));
  const float bias = -slope[0] * 12582912.f;
  const float n = fmaxf(st.m, tile), alpha = exp2f(st.m - n);
  st.m = n;
  if (alpha != 1.f) {
#pragma unroll
    for (int i = 0; i < 4; ++i) { st.out[i][0] *= alpha; st.out[i][1] *= alpha; }
    st.corr *= alpha;
  }
  constexpr float levels = V4 ? 15.f : 255.f;
  const bool any = tile > -CUDART_INF_F;
  float base = any ? tile : n;
  base += tile_base_margin(slope[1], base);
  const float bq = any ? exp2f(base - n) / levels : 0.f, restore = V4 ? bq * (127.f / 7.f) : bq;
  uint32_t w[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float arg = K4 ? fmaf(slope[0], __fsub_rn(x[i], 12582912.f), -base) : fmaf(slope[0], x[i], bias - base);
    const float e = x[i] > -CUDART_INF_F ? exp2f(arg) : 0.f;
    w[i] = __float_as_uint(fmaf(e, levels, x[i] > -CUDART_INF_F ? pmagic_dither(xbits[i]) : 49152.f));
  }
  const uint32_t word = pack_bytes(w[0], w[1], w[2], w[3]);
  pbuf[warp * 32 + lane] = word;
  float part = (float)__dp4a(word, 0x01010101u, 0u) * bq;
  part += __shfl_xor_sync(0xffffffffu, part, 1);
  part += __shfl_xor_sync(0xffffffffu, part, 2);
  st.denom = fmaf(st.denom, alpha, part);
  if constexpr (!V4) st.corr = fmaf(12582912.f, restore, st.corr);
  __syncthreads();
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    int d[4] = {};
#pragma unroll
    for (int kc = 0; kc < 2; ++kc) {
      const uint32_t a0 = pbuf[(2 * kc) * 32 + lane], a2 = pbuf[(2 * kc + 1) * 32 + lane];
      uint32_t b0, b1;
      if constexpr (!V4) {
        const uint32_t* p = reinterpret_cast<const uint32_t*>(vb + (4 * warp + i) * 512 + (2 * kc) * 128 + group * 16 + sub * 4);
        b0 = p[0]; b1 = p[32];
      } else {
        const uint32_t v = *reinterpret_cast<const uint32_t*>(vb + (4 * warp + i) * 256 + kc * 128 + group * 16 + sub * 4);
        b0 = (v << 4) & 0xf0f0f0f0u; b1 = v & 0xf0f0f0f0u;
      }
      mma_u8s8(d, a0, a2, b0, b1);
    }
    if constexpr (!V4) {
      st.out[i][0] = fmaf(__int_as_float(d[0] + Magic), restore, st.out[i][0]);
      st.out[i][1] = fmaf(__int_as_float(d[1] + Magic), restore, st.out[i][1]);
    } else {
      st.out[i][0] = fmaf((float)(d[0] >> 4), restore, st.out[i][0]);
      st.out[i][1] = fmaf((float)(d[1] >> 4), restore, st.out[i][1]);
    }
  }
}

// One 32-key chunk of an un-quantised BF16 head.  Warp w owns keys 8w..8w+7 for QK and channels
// 32w..32w+31 for PV.  Chunk layout: K words [w][feature/16][half][lane], V words
// [channel/8][key/16][half][lane], both in mma.sync B-fragment order.
template <typename AfterSync>
__device__ __forceinline__ void bf16_chunk(const uint8_t* stage, const uint32_t (&qa)[8][2], float sm_log2, uint32_t* pbuf,
    float* rowmax, RowState& st, int key_begin, int prompt, bool row_on, AfterSync after_sync) {
  const int lane = threadIdx.x % 32, warp = threadIdx.x / 32, group = lane / 4, sub = lane % 4;
  const uint32_t* kw = reinterpret_cast<const uint32_t*>(stage);
  const uint32_t* vw = reinterpret_cast<const uint32_t*>(stage + 8192);
  float c[4] = {};
#pragma unroll
  for (int fs = 0; fs < 8; ++fs)
    mma_bf16(c, qa[fs][0], qa[fs][1], kw[((warp * 8 + fs) * 2) * 32 + lane], kw[((warp * 8 + fs) * 2 + 1) * 32 + lane]);
  float s[2];
#pragma unroll
  for (int j = 0; j < 2; ++j) {
    const int key = key_begin + warp * 8 + sub * 2 + j;
    s[j] = (row_on && key < prompt) ? c[j] * sm_log2 : -CUDART_INF_F;
  }
  float mx = fmaxf(s[0], s[1]);
  mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
  mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
  if (sub == 0) rowmax[warp * 8 + group] = mx;
  __syncthreads();
  after_sync();
  const float tile = fmaxf(fmaxf(rowmax[group], rowmax[8 + group]), fmaxf(rowmax[16 + group], rowmax[24 + group]));
  const float n = fmaxf(st.m, tile), alpha = exp2f(st.m - n);
  st.m = n;
  const float p0 = s[0] > -CUDART_INF_F ? exp2f(s[0] - n) : 0.f, p1 = s[1] > -CUDART_INF_F ? exp2f(s[1] - n) : 0.f;
  const __nv_bfloat162 pb = __floats2bfloat162_rn(p0, p1);
  pbuf[warp * 32 + lane] = *reinterpret_cast<const uint32_t*>(&pb);
  float part = p0 + p1;
  part += __shfl_xor_sync(0xffffffffu, part, 1);
  part += __shfl_xor_sync(0xffffffffu, part, 2);
  st.denom = fmaf(st.denom, alpha, part);
  __syncthreads();
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float o[4] = {st.out[i][0] * alpha, st.out[i][1] * alpha, 0.f, 0.f};
    const int cb = 4 * warp + i;
#pragma unroll
    for (int ks = 0; ks < 2; ++ks)
      mma_bf16(o, pbuf[(2 * ks) * 32 + lane], pbuf[(2 * ks + 1) * 32 + lane], vw[((cb * 2 + ks) * 2) * 32 + lane],
               vw[((cb * 2 + ks) * 2 + 1) * 32 + lane]);
    st.out[i][0] = o[0]; st.out[i][1] = o[1];
  }
}

// grid = work items (heaviest first), 128 threads.
// work[w] = {unit, first kept tile, tile count, partial slot}; unit = sequence*heads_kv + kv head.
__global__ void __launch_bounds__(DecodeThreads) decode_kernel(const __nv_bfloat16* q, int64_t qsb, int64_t qsh,
    const uint8_t* pool, const int64_t* unit_base, const int32_t* unit_tab, const int32_t* unit_flags, const int2* tmeta,
    const int4* work, float* pm, float* pl, float* po, int heads_q, int heads_kv, int prompt, float sm_log2, int* err) {
  extern __shared__ __align__(128) uint8_t ring[];
  __shared__ __align__(8) uint64_t full[DecodeStages];
  __shared__ __align__(16) uint8_t qt[MaxGroup * D], qt4[MaxGroup * D];
  __shared__ uint32_t pbuf[2][4 * 32];
  __shared__ int2 smeta[MaxItemTiles];
  __shared__ float rowmax[32], qscale[MaxGroup], qscale4[MaxGroup], dsum[4][8];
  const int tid = threadIdx.x, lane = tid % 32, warp = tid / 32, group = lane / 4, sub = lane % 4;
  const int4 wk = work[blockIdx.x];
  const int unit = wk.x, first = wk.y, count = wk.z, slot = wk.w;
  const int b = unit / heads_kv, kh = unit % heads_kv, g = heads_q / heads_kv;
  const int2* meta = tmeta + unit_tab[unit] + first;
  const uint8_t* base = pool + unit_base[unit];
  const bool bf16 = unit_flags[unit] & 1;
  if (tid == 0) {
#pragma unroll
    for (int s = 0; s < DecodeStages; ++s) mbar_init(&full[s], 1);
    mbar_fence_init();
  }
  for (int i = tid; i < count; i += DecodeThreads) smeta[i] = meta[i];   // the item's tile table, read per tile below
  __syncthreads();
  auto issue = [&](int i) {
    const int2 mt = smeta[i];
    const uint32_t bytes = chunk_bytes((uint32_t)mt.y);
    uint64_t* bar = &full[i % DecodeStages];
    mbar_expect_tx(bar, bytes);
    bulk_g2s(ring + (i % DecodeStages) * StageBytes, base + (int64_t)mt.x * 16, bytes, bar);
  };
  if (tid == 0)
    for (int i = 0; i < DecodeStages - 1 && i < count; ++i) issue(i);

  // Q operands, built while the first chunks are in flight
  const __nv_bfloat16* qrow = q + b * qsb + (int64_t)(kh * g) * qsh;
  uint32_t qf[4][2], qf4[4][2], qb16[8][2];
  if (!bf16) {
    // common_device.cuh:291-315 — same thread mapping as the reference prologue
    for (int r = warp; r < MaxGroup; r += 4) {
      uint32_t word = 0, word4 = 0;
      float mxq = 0.f, xv[4] = {0.f, 0.f, 0.f, 0.f};
      if (r < g) {
        const __nv_bfloat16* src = qrow + r * qsh + lane * 4;
#pragma unroll
        for (int i = 0; i < 4; ++i) xv[i] = __bfloat162float(src[i]);
        rotate128_x4(xv, lane);
#pragma unroll
        for (int i = 0; i < 4; ++i) mxq = fmaxf(mxq, fabsf(xv[i]));
#pragma unroll
        for (int o = 16; o; o >>= 1) mxq = fmaxf(mxq, __shfl_xor_sync(0xffffffffu, mxq, o));
        const float inv = mxq > 0.f ? 127.f / mxq : 0.f, inv4 = mxq > 0.f ? 7.f / mxq : 0.f;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          word |= (uint32_t)(__float2int_rn(xv[i] * inv) & 0xff) << (8 * i);
          word4 |= (uint32_t)((__float2int_rn(xv[i] * inv4) & 0xf) << 4) << (8 * i);   // code * 16 as int8
        }
      }
      reinterpret_cast<uint32_t*>(qt + r * D)[lane] = word;
      reinterpret_cast<uint32_t*>(qt4 + r * D)[lane] = word4;
      if (lane == 0) {
        qscale[r] = r < g ? (mxq > 0.f ? mxq / 127.f * sm_log2 : FLT_MIN) : FLT_MIN;
        qscale4[r] = r < g ? (mxq > 0.f ? mxq / 7.f * sm_log2 : FLT_MIN) : FLT_MIN;
      }
    }
    __syncthreads();
#pragma unroll
    for (int s = 0; s < 4; ++s) {
      qf[s][0] = *reinterpret_cast<const uint32_t*>(qt + group * D + s * 32 + sub * 4);
      qf[s][1] = *reinterpret_cast<const uint32_t*>(qt + group * D + s * 32 + 16 + sub * 4);
      qf4[s][0] = *reinterpret_cast<const uint32_t*>(qt4 + group * D + s * 32 + sub * 4);
      qf4[s][1] = *reinterpret_cast<const uint32_t*>(qt4 + group * D + s * 32 + 16 + sub * 4);
    }
  } else {
#pragma unroll
    for (int fs = 0; fs < 8; ++fs) {
      qb16[fs][0] = group < g ? *reinterpret_cast<const uint32_t*>(qrow + group * qsh + fs * 16 + sub * 2) : 0u;
      qb16[fs][1] = group < g ? *reinterpret_cast<const uint32_t*>(qrow + group * qsh + fs * 16 + 8 + sub * 2) : 0u;
    }
  }
  const float qs8 = bf16 ? 0.f : qscale[group], qs4 = bf16 ? 0.f : qscale4[group];
  RowState st;
  st.m = -FLT_MAX; st.denom = 0.f; st.corr = 0.f;
#pragma unroll
  for (int i = 0; i < 4; ++i) st.out[i][0] = st.out[i][1] = 0.f;

  bool ok = true;
  for (int i = 0; i < count; ++i) {
    // Tile i+3 reuses the stage of tile i-1.  Every thread has finished tile i-1 once it reaches the
    // first barrier of tile i, so the refill is issued right after that barrier; the tile's second
    // barrier orders the rest (pbuf alternates by tile parity), and no third barrier is needed.
    auto refill = [&]() { if (tid == 0 && i + DecodeStages - 1 < count) issue(i + DecodeStages - 1); };
    uint32_t* pb = pbuf[i & 1];
    const int s = i % DecodeStages;
    if (!mbar_wait(&full[s], (i / DecodeStages) & 1)) { ok = false; break; }
    const uint8_t* stage = ring + s * StageBytes;
    const uint32_t info = (uint32_t)smeta[i].y;
    const int tile = info & InfoTileMask;
    const unsigned rowmask = (info >> InfoRowShift) & 0xffu;
    const bool row_on = group < g && ((rowmask >> group) & 1u);
    if (info & InfoBf16) {
      bf16_chunk(stage, qb16, sm_log2, pb, rowmax, st, tile * Bf16ChunkKeys, prompt, row_on, refill);
    } else if (info & InfoK4) {
      if (info & InfoV4) quantised_tile<true, true>(stage, qf4, qs4, pb, rowmax, st, tile * BN, prompt, row_on, refill);
      else quantised_tile<true, false>(stage, qf4, qs4, pb, rowmax, st, tile * BN, prompt, row_on, refill);
    } else {
      if (info & InfoV4) quantised_tile<false, true>(stage, qf, qs8, pb, rowmax, st, tile * BN, prompt, row_on, refill);
      else quantised_tile<false, false>(stage, qf, qs8, pb, rowmax, st, tile * BN, prompt, row_on, refill);
    }
  }
  if (!ok) {
    // A bulk copy never completed.  Record it and leave without touching the outputs; the waits of
    // the other threads run out the same way, so no thread is left behind a barrier.
    if (tid == 0) atomicExch(err, ErrBarrierTimeout);
    return;
  }
  if (sub == 0) dsum[warp][group] = st.denom;
  __syncthreads();
  if (group < g) {
    const int64_t idx = (int64_t)slot * MaxGroup + group;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int ch = warp * 32 + i * 8 + sub * 2;
      *reinterpret_cast<float2*>(po + idx * D + ch) = make_float2(st.out[i][0] - st.corr, st.out[i][1] - st.corr);
    }
    if (warp == 0 && sub == 0) {
      pm[idx] = st.m;
      pl[idx] = dsum[0][group] + dsum[1][group] + dsum[2][group] + dsum[3][group];
    }
  }
}

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
// grid (max kept tiles, units), 256 threads.
__global__ void __launch_bounds__(256) cache_store_kernel(uint8_t* pool, const int64_t* unit_base, const int32_t* unit_tab,
    const int32_t* unit_count, const int32_t* unit_flags, const int2* tmeta, const uint8_t* k8, const uint8_t* k4,
    const float* ka, const float* ka4, const uint8_t* v8, const uint8_t* v4, int tiles) {
  const int i = blockIdx.x, unit = blockIdx.y;
  if (i >= unit_count[unit] || (unit_flags[unit] & 1)) return;
  const int2 mt = tmeta[unit_tab[unit] + i];
  const uint32_t info = (uint32_t)mt.y;
  const int64_t ht = (int64_t)unit * tiles + (info & InfoTileMask);
  uint4* dst = reinterpret_cast<uint4*>(pool + unit_base[unit] + (int64_t)mt.x * 16);
  const bool is_k4 = info & InfoK4, is_v4 = info & InfoV4;
  const int kn = (is_k4 ? K4Bytes : K8Bytes) / 16, vn = (is_v4 ? V4Bytes : V8Bytes) / 16;
  const uint4* ks = reinterpret_cast<const uint4*>(is_k4 ? k4 + ht * K4Bytes : k8 + ht * K8Bytes);
  const uint4* vs = reinterpret_cast<const uint4*>(is_v4 ? v4 + ht * V4Bytes : v8 + ht * V8Bytes);
  for (int j = threadIdx.x; j < kn; j += 256) dst[j] = ks[j];
  for (int j = threadIdx.x; j < vn; j += 256) dst[kn + j] = vs[j];
  if (threadIdx.x == 0) dst[kn + vn] = *reinterpret_cast<const uint4*>((is_k4 ? ka4 : ka) + ht * 4);
}

// grid (32-key chunks, listed BF16 units), 256 threads: K/V bf16 [B,Hkv,T,128] -> fragment-order chunks.
__global__ void __launch_bounds__(256) cache_store_bf16_kernel(uint8_t* pool, const int64_t* unit_base, const int32_t* units,
    const __nv_bfloat16* k, const __nv_bfloat16* v, int tokens, int heads, int64_t ksb, int64_t ksh, int64_t kst, int64_t vsb,
    int64_t vsh, int64_t vst) {
  const int chunk = blockIdx.x, unit = units[blockIdx.y];
  const __nv_bfloat16* kb = k + (unit / heads) * ksb + (unit % heads) * ksh;
  const __nv_bfloat16* vb = v + (unit / heads) * vsb + (unit % heads) * vsh;
  uint32_t* dst = reinterpret_cast<uint32_t*>(pool + unit_base[unit] + (int64_t)chunk * Bf16ChunkBytes);
  const int key0 = chunk * Bf16ChunkKeys;
  for (int w = threadIdx.x; w < 2048; w += 256) {     // K words [nb][fs][half][group][sub]
    const int sub = w % 4, group = (w / 4) % 8, half = (w / 32) % 2, fs = (w / 64) % 8, nb = w / 512;
    const int key = key0 + nb * 8 + group, f = fs * 16 + half * 8 + sub * 2;
    dst[w] = key < tokens ? *reinterpret_cast<const uint32_t*>(kb + (int64_t)key * kst + f) : 0u;
  }
  for (int w = threadIdx.x; w < 2048; w += 256) {     // V words [cb][ks][half][group][sub]
    const int sub = w % 4, group = (w / 4) % 8, half = (w / 32) % 2, ks = (w / 64) % 2, cb = w / 128;
    const int key = key0 + ks * 16 + half * 8 + sub * 2, ch = cb * 8 + group;
    const uint32_t lo = key < tokens ? __bfloat16_as_ushort(vb[(int64_t)key * vst + ch]) : 0u;
    const uint32_t hi = key + 1 < tokens ? __bfloat16_as_ushort(vb[(int64_t)(key + 1) * vst + ch]) : 0u;
    dst[2048 + w] = lo | (hi << 16);
  }
}

static int configure_decode() {
  static int done = 0;   // per process; the attribute is per function and device-independent to set
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
    const int32_t* unit_tab, const int32_t* unit_flags, const int32_t* tmeta, const int32_t* work, int num_work,
    const int32_t* unit_slots, const float* kstat, const float* vstat, void* tail_k, void* tail_v, int64_t tail_stride_u,
    int64_t tail_stride_t, const void* kcur, const void* vcur, int64_t cur_stride_b, int64_t cur_stride_h,
    const int64_t* step, void* out, int64_t out_stride_b, int64_t out_stride_h, float* pm, float* pl, float* po, int batch,
    int heads_q, int heads_kv, int prompt, int max_tail, double scale, int phases, int* device_error, void* stream) {
  TRI_CHECK(q && pool && unit_base && unit_tab && unit_flags && tmeta && work && unit_slots && kstat && vstat && tail_k &&
            tail_v && kcur && vcur && step && out && pm && pl && po && device_error, "decode: null buffers");
  TRI_CHECK(batch > 0 && heads_q > 0 && heads_kv > 0 && heads_q % heads_kv == 0 && heads_q / heads_kv <= MaxGroup &&
            max_tail >= 1 && max_tail <= 1024 && prompt > 0 && num_work >= 0, "decode geometry/buffers");
  // every work item must hold at most MaxItemTiles tiles; the host planner guarantees it (checked there)
  TRI_CHECK(aligned16(pool) && aligned16(po) && (reinterpret_cast<uintptr_t>(q) & 7u) == 0 && q_stride_b % 4 == 0 &&
            q_stride_h % 4 == 0, "decode: alignment");
  if (configure_decode() != TRI_OK) return TRI_ERR_CUDA;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const float sm_log2 = (float)(scale * 1.4426950408889634);
  const auto* qp = static_cast<const __nv_bfloat16*>(q);
  if (num_work > 0 && (phases & 1))
    decode_kernel<<<num_work, DecodeThreads, DecodeShared, s>>>(qp, q_stride_b, q_stride_h, static_cast<const uint8_t*>(pool),
        unit_base, unit_tab, unit_flags, reinterpret_cast<const int2*>(tmeta), reinterpret_cast<const int4*>(work), pm, pl, po,
        heads_q, heads_kv, prompt, sm_log2, device_error);
  if (phases & 2)
    decode_merge_kernel<<<dim3(heads_q, batch), MergeThreads, 0, s>>>(pm, pl, po, reinterpret_cast<const int2*>(unit_slots), vstat,
      kstat, qp, q_stride_b, q_stride_h, static_cast<__nv_bfloat16*>(tail_k), static_cast<__nv_bfloat16*>(tail_v),
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
    int64_t v_stride_h, int64_t v_stride_t, void* stream) {
  TRI_CHECK(pool && unit_base && units && k && v && num_units > 0 && tokens > 0 && heads_kv > 0, "cache_store_bf16: arguments");
  TRI_CHECK(k_stride_t % 2 == 0 && k_stride_h % 2 == 0 && k_stride_b % 2 == 0 && (reinterpret_cast<uintptr_t>(k) & 3u) == 0,
            "cache_store_bf16: K rows must be 4-byte aligned");
  const int chunks = (tokens + Bf16ChunkKeys - 1) / Bf16ChunkKeys;
  cache_store_bf16_kernel<<<dim3(chunks, num_units), 256, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<uint8_t*>(pool),
      unit_base, units, static_cast<const __nv_bfloat16*>(k), static_cast<const __nv_bfloat16*>(v), tokens, heads_kv,
      k_stride_b, k_stride_h, k_stride_t, v_stride_b, v_stride_h, v_stride_t);
  return tri_launch_status("cache_store_bf16");
}
