// KV-cache write path for sm_100a: channel statistics, then fused rotate + quantise + pack.
//
// Replaces (paths inside the reference project)
//   triattention/kernels/cuda/common_device.cuh:1-28     quantize_q_kernel
//   triattention/kernels/cuda/common_device.cuh:32-56    partial_kernel, finalize_kernel
//   triattention/kernels/cuda/common_device.cuh:58-131   quantize_k_kernel
//   triattention/kernels/cuda/common_device.cuh:132-172  pack_v_kernel
//   triattention/kernels/cuda/common_host.cuh:1-45       prepare_qk, pack_v host launchers
// with a batch dimension added (the reference is batch 1).  Float operation order is kept where the
// result bits depend on it: the 64-way strided partial sums, their in-order total, the butterflies of
// the rotation, and the scale expressions.
//
// Design: everything here is HBM-bound byte work.  The Walsh-Hadamard transform runs in registers:
// Q rows with 32 features per lane (4 lanes per row: 5 in-register radix-2 stages, 2 shuffle stages), K rows
// with 16 features per lane (8 lanes per row: 4 in-register stages, 3 shuffle stages), so every lane ends up
// owning whole 16-byte runs of codes and stores them with 128-bit stores.
// K needs the whole-prompt channel mean and V the whole-prompt mean and range before any code can be
// produced, so the write is two phases: statistics (K and V together), then codes (K, V).
#include "common.cuh"
#include "abi_internal.h"

namespace tri {

// ------------------------------------------------------------------------------------------------
// statistics: partial[tensor][unit][block][3][128], stat[unit][3][128]
// ------------------------------------------------------------------------------------------------
// grid (StatBlocks, units, 2 tensors), 128 threads = one per channel.  Block b owns tokens b, b+64, ...
// and adds them in token order (common_device.cuh:36-39): the order is part of the mean's bit pattern.
__global__ void __launch_bounds__(D) stats_partial_kernel(const __nv_bfloat16* k, const __nv_bfloat16* v,
    float* partial_k, float* partial_v, int tokens, int heads, int64_t ksb, int64_t ksh, int64_t kst,
    int64_t vsb, int64_t vsh, int64_t vst) {
  grid_dependency_wait();     // launched with launch_chained(): nothing is read or written before the predecessor is done
  grid_launch_dependents();
  const int c = threadIdx.x, unit = blockIdx.y, which = blockIdx.z;
  const int b = unit / heads, h = unit % heads;
  const __nv_bfloat16* base;
  int64_t st;
  float* partial;
  if (which == 0) {
    if (k == nullptr) return;
    base = k + b * ksb + h * ksh + c; st = kst; partial = partial_k;
  } else {
    if (v == nullptr) return;
    base = v + b * vsb + h * vsh + c; st = vst; partial = partial_v;
  }
  float sum = 0.f, hi = -FLT_MAX, lo = FLT_MAX;
  int t = blockIdx.x;
  // loads are issued 32 at a time (the kernel is bound by their latency); the adds stay sequential in token order
  for (; t + 31 * StatBlocks < tokens; t += 32 * StatBlocks) {
    float x[32];
#pragma unroll
    for (int u = 0; u < 32; ++u) x[u] = __bfloat162float(base[(int64_t)(t + u * StatBlocks) * st]);
#pragma unroll
    for (int u = 0; u < 32; ++u) { sum += x[u]; hi = fmaxf(hi, x[u]); lo = fminf(lo, x[u]); }
  }
  for (; t + 7 * StatBlocks < tokens; t += 8 * StatBlocks) {
    float x[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) x[u] = __bfloat162float(base[(int64_t)(t + u * StatBlocks) * st]);
#pragma unroll
    for (int u = 0; u < 8; ++u) { sum += x[u]; hi = fmaxf(hi, x[u]); lo = fminf(lo, x[u]); }
  }
  for (; t < tokens; t += StatBlocks) {
    const float x = __bfloat162float(base[(int64_t)t * st]);
    sum += x; hi = fmaxf(hi, x); lo = fminf(lo, x);
  }
  float* o = partial + (((int64_t)unit * StatBlocks + blockIdx.x) * 3) * D + c;
  o[0] = sum; o[D] = hi; o[2 * D] = lo;
}

// grid (units, 2), 128 threads.  common_device.cuh:44-56.
__global__ void __launch_bounds__(D) stats_finalize_kernel(const float* partial_k, const float* partial_v,
    float* kstat, float* vstat, int tokens, int v_identity, const int32_t* raw_heads, int heads) {
  grid_dependency_wait();     // launched with launch_chained(): nothing is read or written before the predecessor is done
  grid_launch_dependents();
  const int64_t unit = blockIdx.x;
  const int c = threadIdx.x, which = blockIdx.y;
  const float* partial = which == 0 ? partial_k : partial_v;
  float* stat = which == 0 ? kstat : vstat;
  if (stat == nullptr) return;
  float mean = 0.f, scale = 1.f;
  // V of an un-quantised head stays as it is: identity statistics (0, 1, 1), like the reference's identity mode
  const bool identity = which == 1 && (v_identity || (raw_heads != nullptr && raw_heads[unit % heads] != 0));
  if (!identity) {
    const float* in = partial + unit * StatBlocks * 3 * D + c;
    float sum = 0.f, hi = -FLT_MAX, lo = FLT_MAX;
    for (int b0 = 0; b0 < StatBlocks; b0 += 16) {   // 48 loads in flight; the sum stays sequential in block order
      float ps[16], ph[16], pl[16];
#pragma unroll
      for (int u = 0; u < 16; ++u) {
        ps[u] = in[(b0 + u) * 3 * D]; ph[u] = in[(b0 + u) * 3 * D + D]; pl[u] = in[(b0 + u) * 3 * D + 2 * D];
      }
#pragma unroll
      for (int u = 0; u < 16; ++u) { sum += ps[u]; hi = fmaxf(hi, ph[u]); lo = fminf(lo, pl[u]); }
    }
    mean = sum / tokens;
    const float range = fmaxf(hi - mean, mean - lo);
    scale = range > 0.f ? range / 127.f : 1.f;
  }
  stat[unit * 3 * D + c] = mean; stat[unit * 3 * D + D + c] = scale; stat[unit * 3 * D + 2 * D + c] = 1.f / scale;
}

// ------------------------------------------------------------------------------------------------
// Q: rotate, per-token absmax, INT8 codes + INT4 codes (as int8 values), scales
// ------------------------------------------------------------------------------------------------
__device__ __forceinline__ void load16_bf16(const __nv_bfloat16* src, float (&x)[16]) {
  const uint4 a = *reinterpret_cast<const uint4*>(src), b = *reinterpret_cast<const uint4*>(src + 8);
  const uint32_t w[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    x[2 * i] = __uint_as_float(w[i] << 16);
    x[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}
// rn_even(p) & 0xff for |p| < 2^22 without the conversion unit: p + 12582912.0f rounds p to an integer exactly like
// cvt.rni (one rounding, ties to even), and the low byte of the sum's bit pattern is the two's-complement code.
__device__ __forceinline__ uint32_t rn_bits(float p) { return __float_as_uint(__fadd_rn(p, 12582912.f)); }
__device__ __forceinline__ uint32_t pack_low_bytes(uint32_t w0, uint32_t w1, uint32_t w2, uint32_t w3) {
  return __byte_perm(__byte_perm(w0, w1, 0x0040), __byte_perm(w2, w3, 0x0040), 0x5410);
}
// 16 codes rn_even(x * inv) as bytes: the product is rounded to fp32 first (a separate multiply, as in the
// reference's __float2int_rn(x * inv), common_device.cuh:14), then to an integer.
__device__ __forceinline__ uint4 codes16(const float (&x)[16], float inv) {
  uint32_t w[4];
#pragma unroll
  for (int j = 0; j < 4; ++j)
    w[j] = pack_low_bytes(rn_bits(__fmul_rn(x[4 * j], inv)), rn_bits(__fmul_rn(x[4 * j + 1], inv)),
                          rn_bits(__fmul_rn(x[4 * j + 2], inv)), rn_bits(__fmul_rn(x[4 * j + 3], inv)));
  return make_uint4(w[0], w[1], w[2], w[3]);
}

// A lane of quantize_q_kernel holds two runs of 16 features, 16*(l4 + 4k) .. +15 for k = 0, 1, as 8 bf16 pairs
// each.  Sign flips of the rotation for them: word 8k+j flips bit 15 if the run's feature 2j is negated and bit 31
// if feature 2j+1 is (the sign words of prefill_sm80.cu:27).
struct PairSigns { uint32_t w[4][16]; };
constexpr PairSigns make_pair_signs() {
  constexpr uint32_t words[4] = {0x9a3b5e71u, 0x2c6d8f13u, 0xe41b7a95u, 0x5f02c3d8u};
  PairSigns t{};
  for (int l = 0; l < 4; ++l)
    for (int k = 0; k < 2; ++k)
      for (int j = 0; j < 8; ++j) {
        const int f = 16 * (l + 4 * k) + 2 * j;
        t.w[l][8 * k + j] = (((words[f >> 5] >> (f & 31)) & 1u) << 15) | (((words[(f + 1) >> 5] >> ((f + 1) & 31)) & 1u) << 31);
      }
  return t;
}
__device__ const PairSigns kPairSigns = make_pair_signs();

// grid (ceil(T/32), B*Hq), 128 threads: 8 rows per warp, 4 lanes per row, 32 features per lane.  The lane index is
// feature bits 4-5: butterflies on bits 0-3 in registers, bits 4-5 across lanes, bit 6 in registers again (the same
// butterflies in the same order as rotate128_x16, so the same bits).  With this assignment the four lanes of a
// row read 128 contiguous bytes per load and write 64 contiguous bytes per store.
// The kernel is bound by the SM's load/store data path (shuffles, 16-byte global accesses) and by instruction
// issue, not by HBM: 32 features per lane need 22 instructions and 8 shuffles per row-warp where 16 features
// needed 28 and 12; a whole row per thread needs no shuffle, but its global accesses no longer coalesce and its
// 159 registers leave too few warps.
// q8/q4x are plain [B*Hq][T][128] int8 (the reference's q8 layout, common_device.cuh:18); q4x holds the 4-bit
// codes sign-extended to int8 so that the prefill kernel can feed them to the INT8 tensor-core path.
__global__ void __launch_bounds__(128) quantize_q_kernel(const __nv_bfloat16* q, int8_t* q8, float* qa, int8_t* q4x,
    float* qa4, const int32_t* q_modes, int tokens, int heads, int64_t qsb, int64_t qsh, int64_t qst) {
  grid_dependency_wait();     // launched with launch_chained(): nothing is read or written before the predecessor is done
  grid_launch_dependents();
  const int lane = threadIdx.x % 32, l4 = lane % 4;
  const int row = blockIdx.x * 32 + (threadIdx.x / 32) * 8 + lane / 4;
  const int unit = blockIdx.y;
  // what the attention will read of this head: bit 0 = INT8 codes, bit 1 = INT4 codes (a head without an INT4 band
  // needs none, an un-quantised head neither)
  const int mode = q_modes != nullptr ? q_modes[unit % heads] : 3;
  if (!(mode & 1)) return;
  if (!(mode & 2)) q4x = nullptr;
  const bool live = row < tokens;
  float x[32];   // x[16k + e] = feature 16*(l4 + 4k) + e
  {
    const __nv_bfloat16* src = q + (unit / heads) * qsb + (unit % heads) * qsh + (int64_t)row * qst + l4 * 16;
    const uint4* flip = reinterpret_cast<const uint4*>(kPairSigns.w[l4]);
#pragma unroll
    for (int i = 0; i < 4; ++i) {          // 16-byte piece i: run k = i/2, features 8*(i%2) .. +7 of it
      const uint4 a = live ? *reinterpret_cast<const uint4*>(src + (i / 2) * 64 + (i % 2) * 8) : make_uint4(0, 0, 0, 0);
      const uint4 f = flip[i];
      const uint32_t w[4] = {a.x ^ f.x, a.y ^ f.y, a.z ^ f.z, a.w ^ f.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        x[8 * i + 2 * j] = __uint_as_float(w[j] << 16);
        x[8 * i + 2 * j + 1] = __uint_as_float(w[j] & 0xffff0000u);
      }
    }
  }
  auto in_registers = [&](int bit) {
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      if (!(i & bit)) {
        const float lo = x[i], hi = x[i | bit];
        x[i] = lo + hi; x[i | bit] = lo - hi;
      }
    }
  };
  in_registers(1); in_registers(2); in_registers(4); in_registers(8);          // feature bits 0-3
#pragma unroll
  for (int bit = 1; bit < 4; bit <<= 1) {                                       // feature bits 4-5
    const float sign = (l4 & bit) ? -1.f : 1.f;   // upper lane: partner - own; lower lane: own + partner
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      const float y = __shfl_xor_sync(0xffffffffu, x[i], bit);
      x[i] = fmaf(x[i], sign, y);                 // one rounding of y +- x, like the add / subtract it replaces
    }
  }
  in_registers(16);                                                             // feature bit 6
  float m0 = 0.f, m1 = 0.f;
#pragma unroll
  for (int i = 0; i < 32; i += 2) {
    x[i] *= kRotScale; x[i + 1] *= kRotScale;
    m0 = fmaxf(m0, fabsf(x[i])); m1 = fmaxf(m1, fabsf(x[i + 1]));
  }
  float m = fmaxf(m0, m1);
  m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 1));
  m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 2));
  if (!live) return;
  const int64_t r = (int64_t)unit * tokens + row;
  const float inv = m > 0.f ? 127.f / m : 0.f;
  int8_t* d8 = q8 + r * D + l4 * 16;
  *reinterpret_cast<uint4*>(d8) = codes16(reinterpret_cast<const float(&)[16]>(x[0]), inv);
  *reinterpret_cast<uint4*>(d8 + 64) = codes16(reinterpret_cast<const float(&)[16]>(x[16]), inv);
  if (l4 == 0) qa[r] = m / 127.f;
  if (q4x != nullptr) {
    const float inv4 = m > 0.f ? 7.f / m : 0.f;
    int8_t* d4 = q4x + r * D + l4 * 16;
    *reinterpret_cast<uint4*>(d4) = codes16(reinterpret_cast<const float(&)[16]>(x[0]), inv4);
    *reinterpret_cast<uint4*>(d4 + 64) = codes16(reinterpret_cast<const float(&)[16]>(x[16]), inv4);
    if (l4 == 0) qa4[r] = m / 7.f;
  }
}

// ------------------------------------------------------------------------------------------------
// K: centre, rotate, per-16-key absmax, INT8 / INT4 codes into tile blobs
// ------------------------------------------------------------------------------------------------
// grid (tiles, B*Hkv), 128 threads.  One warp owns one 16-key scale group end to end, so no block
// barrier is needed: 4 passes of 4 rows, 64 rotated values kept in registers until the group
// maximum is known.
__global__ void __launch_bounds__(128) quantize_k_kernel(const __nv_bfloat16* k, const float* kstat, uint8_t* k8,
    float* ka, uint8_t* k4x, uint8_t* k4, float* ka4, int tokens, int heads, int64_t ksb, int64_t ksh, int64_t kst) {
  grid_dependency_wait();     // launched with launch_chained(): nothing is read or written before the predecessor is done
  grid_launch_dependents();
  const int tile = blockIdx.x, unit = blockIdx.y, tiles = gridDim.x;
  const int col = threadIdx.x / 32, lane = threadIdx.x % 32, l8 = lane % 8, sub_row = lane / 8;
  const __nv_bfloat16* src = k + (unit / heads) * ksb + (unit % heads) * ksh + l8 * 16;
  float mean[16];
  {
    const float4* mp = reinterpret_cast<const float4*>(kstat + (int64_t)unit * StatFloats + l8 * 16);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float4 v = mp[i];
      mean[4 * i] = v.x; mean[4 * i + 1] = v.y; mean[4 * i + 2] = v.z; mean[4 * i + 3] = v.w;
    }
  }
  float y[4][16];
  float cm = 0.f;
#pragma unroll
  for (int p = 0; p < 4; ++p) {
    const int t = tile * BN + col * 16 + p * 4 + sub_row;
    if (t < tokens) {
      load16_bf16(src + (int64_t)t * kst, y[p]);
#pragma unroll
      for (int i = 0; i < 16; ++i) y[p][i] -= mean[i];
    } else {
#pragma unroll
      for (int i = 0; i < 16; ++i) y[p][i] = 0.f;
    }
    rotate128_x16(y[p], l8);
#pragma unroll
    for (int i = 0; i < 16; ++i) cm = fmaxf(cm, fabsf(y[p][i]));
  }
#pragma unroll
  for (int o = 16; o; o >>= 1) cm = fmaxf(cm, __shfl_xor_sync(0xffffffffu, cm, o));
  const float inv = cm > 0.f ? 127.f / cm : 0.f, inv4 = cm > 0.f ? 7.f / cm : 0.f;
  const int64_t ht = (int64_t)unit * tiles + tile;
  if (lane == 0) {
    ka[ht * 4 + col] = cm > 0.f ? cm / 127.f : 1.f;
    if (ka4 != nullptr) ka4[ht * 4 + col] = cm > 0.f ? cm / 7.f : 1.f;
  }
#pragma unroll
  for (int p = 0; p < 4; ++p) {
    const int r = col * 16 + p * 4 + sub_row;            // key row inside the tile
    const int core = (r / 8) * 1024 + l8 * 128 + (r % 8) * 16;
    *reinterpret_cast<uint4*>(k8 + ht * K8Bytes + core) = codes16(y[p], inv);
    if (k4x == nullptr && k4 == nullptr) continue;
    const uint4 c4 = codes16(y[p], inv4);
    if (k4x != nullptr) *reinterpret_cast<uint4*>(k4x + ht * K8Bytes + core) = c4;
    if (k4 != nullptr) {
      // decode layout [key/8][key%8][sub][16 B]: this lane owns features 32*sub + 16*h + 0..15 and writes
      // words s = 2h, 2h+1 of the run; byte j of word s: low nibble = feature 32*sub+8s+j, high = +4
      const uint32_t lo = (c4.x & 0x0f0f0f0fu) | ((c4.y & 0x0f0f0f0fu) << 4);
      const uint32_t hi = (c4.z & 0x0f0f0f0fu) | ((c4.w & 0x0f0f0f0fu) << 4);
      *reinterpret_cast<uint2*>(k4 + ht * K4Bytes + (r / 8) * 512 + (r % 8) * 64 + (l8 >> 1) * 16 + (l8 & 1) * 8) = make_uint2(lo, hi);
    }
  }
}

// ------------------------------------------------------------------------------------------------
// V: per-channel affine normalise, FP16 / INT8 / INT4 tile blobs (channel-major, keys contiguous)
// ------------------------------------------------------------------------------------------------
// grid (tiles, B*Hkv), 256 threads.  The tile is transposed through shared memory once; each thread
// then emits whole 16-byte runs.
__global__ void __launch_bounds__(256) pack_v_kernel(const __nv_bfloat16* v, const float* vstat, uint8_t* v16,
    uint8_t* v8, uint8_t* v4, uint8_t* v8h, int tokens, int heads, int64_t vsb, int64_t vsh, int64_t vst,
    const int32_t* raw_heads) {
  // Row stride 132 floats: a thread stores its 8 channels of a row as two 16-byte words (two lanes of a quarter
  // warp share a bank), and a warp that later reads 32 consecutive channels of one row hits 32 different banks.
  __shared__ __align__(16) float vn[BN][D + 4];
  grid_dependency_wait();     // launched with launch_chained(): nothing is read or written before the predecessor is done
  grid_launch_dependents();
  const int tile = blockIdx.x, unit = blockIdx.y, tiles = gridDim.x, tid = threadIdx.x;
  const __nv_bfloat16* base = v + (unit / heads) * vsb + (unit % heads) * vsh;
  const float* stat = vstat + (int64_t)unit * StatFloats;
  // an un-quantised head gets only the fp16 blob (its statistics are the identity, so V' = V), with values beyond the
  // fp16 range clamped to +-65504; no integer codes
  const bool raw_unit = raw_heads != nullptr && raw_heads[unit % heads] != 0;
  if (raw_unit) { v8 = nullptr; v4 = nullptr; v8h = nullptr; }
  {
    const int c0 = (tid % (D / 8)) * 8;     // the same 8 channels in every pass
    float mean[8], inv[8];
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const float4 m = *reinterpret_cast<const float4*>(stat + c0 + 4 * j);
      const float4 s = *reinterpret_cast<const float4*>(stat + 2 * D + c0 + 4 * j);
      mean[4 * j] = m.x; mean[4 * j + 1] = m.y; mean[4 * j + 2] = m.z; mean[4 * j + 3] = m.w;
      inv[4 * j] = s.x; inv[4 * j + 1] = s.y; inv[4 * j + 2] = s.z; inv[4 * j + 3] = s.w;
    }
#pragma unroll
    for (int pass = 0; pass < BN * D / 8 / 256; ++pass) {
      const int r = pass * (256 / (D / 8)) + tid / (D / 8), t = tile * BN + r;
      float y[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      if (t < tokens) {
        const uint4 raw = *reinterpret_cast<const uint4*>(base + (int64_t)t * vst + c0);
        const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          // vnorm, common_device.cuh:132-134: (v - mean) * (1/scale)
          y[2 * j] = (__uint_as_float(w[j] << 16) - mean[2 * j]) * inv[2 * j];
          y[2 * j + 1] = (__uint_as_float(w[j] & 0xffff0000u) - mean[2 * j + 1]) * inv[2 * j + 1];
        }
      }
      *reinterpret_cast<float4*>(&vn[r][c0]) = make_float4(y[0], y[1], y[2], y[3]);
      *reinterpret_cast<float4*>(&vn[r][c0 + 4]) = make_float4(y[4], y[5], y[6], y[7]);
    }
  }
  __syncthreads();
  const int64_t ht = (int64_t)unit * tiles + tile;
  // One thread = one channel and 32 keys, read from the transposed tile once for every output format
  // (run = 16 bytes of a blob: 8 keys of a channel in V16 / V8H, 16 keys in V8, 32 keys in V4).
  // (a warp holds 32 consecutive channels of one key half, so its reads of a row hit 32 different banks)
  const int ch = tid % D, kc = tid / D;
  float x[32];
#pragma unroll
  for (int kk = 0; kk < 32; ++kk) x[kk] = vn[kc * 32 + kk][ch];
  if (raw_unit) {
#pragma unroll
    for (int kk = 0; kk < 32; ++kk) x[kk] = fminf(fmaxf(x[kk], -65504.f), 65504.f);
  }
  if (v16 != nullptr) {
#pragma unroll
    for (int q = 0; q < 4; ++q) {          // run (ch/8, key/8, ch%8)
      uint32_t w[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const __half2 h = __floats2half2_rn(x[8 * q + 2 * j], x[8 * q + 2 * j + 1]);
        w[j] = *reinterpret_cast<const uint32_t*>(&h);
      }
      const int run = (ch / 8) * 64 + (kc * 4 + q) * 8 + ch % 8;
      *reinterpret_cast<uint4*>(v16 + ht * V16Bytes + (int64_t)run * 16) = make_uint4(w[0], w[1], w[2], w[3]);
    }
  }
  if (v8 != nullptr || v8h != nullptr) {
    // clamp(rn(x)) == rn(clamp(x)): rounding is monotonic and the bounds are integers.  c[kk] = 12582912 + code as
    // float bits: the low byte is the INT8 code, and minus 12582912.0f it is the code as a float.
    uint32_t c[32];
#pragma unroll
    for (int kk = 0; kk < 32; ++kk) c[kk] = rn_bits(fminf(fmaxf(x[kk], -127.f), 127.f));
    if (v8h != nullptr) {
      // The INT8 codes once more, as fp16 numbers in the V16 layout: the P.V operand of the tcgen05 prefill, whose
      // weights are fp16.
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        uint32_t w[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const __half2 h = __floats2half2_rn(__fadd_rn(__uint_as_float(c[8 * q + 2 * j]), -12582912.f),
                                              __fadd_rn(__uint_as_float(c[8 * q + 2 * j + 1]), -12582912.f));
          w[j] = *reinterpret_cast<const uint32_t*>(&h);
        }
        const int run = (ch / 8) * 64 + (kc * 4 + q) * 8 + ch % 8;
        *reinterpret_cast<uint4*>(v8h + ht * V16Bytes + (int64_t)run * 16) = make_uint4(w[0], w[1], w[2], w[3]);
      }
    }
    if (v8 != nullptr) {
#pragma unroll
      for (int h = 0; h < 2; ++h) {        // run (ch/8, key/16, ch%8): 16 keys in kperm order
        uint32_t w[4];
#pragma unroll
        for (int s = 0; s < 4; ++s)
          w[s] = pack_low_bytes(c[16 * h + kperm(s, 0)], c[16 * h + kperm(s, 1)], c[16 * h + kperm(s, 2)], c[16 * h + kperm(s, 3)]);
        const int run = (ch / 8) * 32 + (kc * 2 + h) * 8 + ch % 8;
        *reinterpret_cast<uint4*>(v8 + ht * V8Bytes + (int64_t)run * 16) = make_uint4(w[0], w[1], w[2], w[3]);
      }
    }
  }
  if (v4 != nullptr) {                     // run (ch/8, key/32, ch%8): 32 keys, two per byte
    uint32_t w[4];
#pragma unroll
    for (int s = 0; s < 4; ++s) {
      uint32_t word = 0;
#pragma unroll
      for (int b = 0; b < 4; ++b) {
        const uint32_t lo = rn_bits(fminf(fmaxf(__fmul_rn(x[kperm(s, b)], 7.f / 127.f), -7.f), 7.f));
        const uint32_t hi = rn_bits(fminf(fmaxf(__fmul_rn(x[16 + kperm(s, b)], 7.f / 127.f), -7.f), 7.f));
        word |= ((lo & 0xfu) | ((hi & 0xfu) << 4)) << (8 * b);
      }
      w[s] = word;
    }
    const int run = (ch / 8) * 16 + kc * 8 + ch % 8;
    *reinterpret_cast<uint4*>(v4 + ht * V4Bytes + (int64_t)run * 16) = make_uint4(w[0], w[1], w[2], w[3]);
  }
}

}  // namespace tri

using namespace tri;

// ---- argument checks and launch chains shared by the entry points --------------------------------------------------
struct QkArgs {
  const void *q, *k;
  int batch, heads_q, heads_kv, tokens;
  int64_t qsb, qsh, qst, ksb, ksh, kst;
  void* q8; float* qa; void* k8; float* ka; float* partial; float* kstat;
  void* q4x; float* qa4; void* k4x; void* k4; float* ka4; const int32_t* q_modes;
};
struct VArgs {
  const void* v;
  int batch, heads_kv, tokens;
  int64_t vsb, vsh, vst;
  float* partial; float* vstat; void *v16, *v8, *v4, *v8h; const int32_t* raw_heads;
};

static int check_qk(const QkArgs& a) {
  TRI_CHECK(a.q && a.k && a.q8 && a.qa && a.k8 && a.ka && a.partial && a.kstat, "prepare_qk: null Q/K buffers");
  TRI_CHECK(a.batch > 0 && a.heads_q > 0 && a.heads_kv > 0 && a.tokens > 0 && a.heads_q % a.heads_kv == 0, "prepare_qk: bad geometry");
  TRI_CHECK((a.tokens + BN - 1) / BN <= MaxTiles, "at most 131072 tokens");
  const bool int4 = a.q4x != nullptr;
  TRI_CHECK(int4 == (a.qa4 != nullptr) && int4 == (a.k4x != nullptr) && int4 == (a.ka4 != nullptr) && (int4 || a.k4 == nullptr),
            "INT4 Q/K buffers (all or none)");
  TRI_CHECK(aligned16(a.q) && aligned16(a.k) && a.qsb % 8 == 0 && a.qsh % 8 == 0 && a.qst % 8 == 0 && a.ksb % 8 == 0 &&
            a.ksh % 8 == 0 && a.kst % 8 == 0, "BF16 Q/K [B,H,T,128] with contiguous features, 16-byte aligned rows");
  TRI_CHECK(aligned16(a.q8) && aligned16(a.k8) && aligned16(a.q4x) && aligned16(a.k4x) && aligned16(a.k4) && aligned16(a.kstat),
            "prepare_qk: output buffers must be 16-byte aligned");
  return TRI_OK;
}
static int check_v(const VArgs& a) {
  TRI_CHECK(a.v && a.partial && a.vstat, "pack_v: null V buffers");
  TRI_CHECK(a.batch > 0 && a.heads_kv > 0 && a.tokens > 0, "pack_v: bad geometry");
  TRI_CHECK(aligned16(a.v) && a.vsb % 8 == 0 && a.vsh % 8 == 0 && a.vst % 8 == 0, "BF16 V [B,Hkv,T,128]");
  TRI_CHECK(aligned16(a.v16) && aligned16(a.v8) && aligned16(a.v4) && aligned16(a.v8h) && aligned16(a.vstat), "packed V alignment");
  return TRI_OK;
}
// the three chains are independent of one another: Q (one kernel), K (statistics, then codes), V (statistics, then blobs)
static void launch_q(const QkArgs& a, cudaStream_t s) {
  launch_chained(quantize_q_kernel, dim3((a.tokens + 31) / 32, a.batch * a.heads_q), dim3(128), 0, s,
      static_cast<const __nv_bfloat16*>(a.q), static_cast<int8_t*>(a.q8), a.qa, static_cast<int8_t*>(a.q4x), a.qa4, a.q_modes,
      a.tokens, a.heads_q, a.qsb, a.qsh, a.qst);
}
static void launch_k(const QkArgs& a, cudaStream_t s) {
  const int tiles = (a.tokens + BN - 1) / BN, uk = a.batch * a.heads_kv;
  const auto* kp = static_cast<const __nv_bfloat16*>(a.k);
  launch_chained(stats_partial_kernel, dim3(StatBlocks, uk, 1), dim3(D), 0, s, kp, nullptr, a.partial, nullptr, a.tokens, a.heads_kv,
      a.ksb, a.ksh, a.kst, 0, 0, 0);
  launch_chained(stats_finalize_kernel, dim3(uk, 1), dim3(D), 0, s, a.partial, nullptr, a.kstat, nullptr, a.tokens, 0,
      static_cast<const int32_t*>(nullptr), a.heads_kv);
  launch_chained(quantize_k_kernel, dim3(tiles, uk), dim3(128), 0, s, kp, a.kstat, static_cast<uint8_t*>(a.k8), a.ka,
      static_cast<uint8_t*>(a.k4x), static_cast<uint8_t*>(a.k4), a.ka4, a.tokens, a.heads_kv, a.ksb, a.ksh, a.kst);
}
static void launch_v(const VArgs& a, cudaStream_t s) {
  const int tiles = (a.tokens + BN - 1) / BN, uk = a.batch * a.heads_kv;
  const auto* vp = static_cast<const __nv_bfloat16*>(a.v);
  const int identity = (a.v8 == nullptr && a.v4 == nullptr && a.v8h == nullptr) ? 1 : 0;  // common_host.cuh:39
  if (!identity)
    launch_chained(stats_partial_kernel, dim3(StatBlocks, uk, 2), dim3(D), 0, s, nullptr, vp, nullptr, a.partial, a.tokens, a.heads_kv,
        0, 0, 0, a.vsb, a.vsh, a.vst);
  launch_chained(stats_finalize_kernel, dim3(uk, 2), dim3(D), 0, s, nullptr, a.partial, nullptr, a.vstat, a.tokens, identity,
      a.raw_heads, a.heads_kv);
  launch_chained(pack_v_kernel, dim3(tiles, uk), dim3(256), 0, s, vp, a.vstat, static_cast<uint8_t*>(a.v16), static_cast<uint8_t*>(a.v8),
      static_cast<uint8_t*>(a.v4), static_cast<uint8_t*>(a.v8h), a.tokens, a.heads_kv, a.vsb, a.vsh, a.vst, a.raw_heads);
}

// Two side streams and three events per device for tri_write_kv, made on first use.  The mutex is held from the fork to
// the join of one call, so that two host threads never re-record an event the other is still waiting on.
#include <mutex>
struct WriteLanes {
  std::mutex lock;
  bool ready = false;
  cudaStream_t side[2];
  cudaEvent_t fork, join[2];
};
static WriteLanes g_lanes[TriPerDevice::MaxDevices];

// ------------------------------------------------------------------------------------------------
// C ABI
// ------------------------------------------------------------------------------------------------
extern "C" int tri_prepare_qk(const void* q, const void* k, int batch, int heads_q, int heads_kv, int tokens,
    int64_t q_stride_b, int64_t q_stride_h, int64_t q_stride_t, int64_t k_stride_b, int64_t k_stride_h,
    int64_t k_stride_t, void* q8, float* qa, void* k8, float* ka, float* partial, float* kstat, void* q4x,
    float* qa4, void* k4x, void* k4, float* ka4, const int32_t* q_modes, void* stream) {
  const QkArgs a{q, k, batch, heads_q, heads_kv, tokens, q_stride_b, q_stride_h, q_stride_t, k_stride_b, k_stride_h, k_stride_t,
                 q8, qa, k8, ka, partial, kstat, q4x, qa4, k4x, k4, ka4, q_modes};
  if (const int rc = check_qk(a)) return rc;
  launch_q(a, static_cast<cudaStream_t>(stream));
  launch_k(a, static_cast<cudaStream_t>(stream));
  return tri_launch_status("prepare_qk");
}

extern "C" int tri_pack_v(const void* v, int batch, int heads_kv, int tokens, int64_t v_stride_b, int64_t v_stride_h,
    int64_t v_stride_t, float* partial, float* vstat, void* v16, void* v8, void* v4, void* v8h, const int32_t* raw_heads,
    void* stream) {
  const VArgs a{v, batch, heads_kv, tokens, v_stride_b, v_stride_h, v_stride_t, partial, vstat, v16, v8, v4, v8h, raw_heads};
  if (const int rc = check_v(a)) return rc;
  launch_v(a, static_cast<cudaStream_t>(stream));
  return tri_launch_status("pack_v");
}

// tri_prepare_qk and tri_pack_v as one call whose three chains run side by side: the Q kernel on the caller's stream, the
// K and V chains on two high-priority streams of the library that start behind everything already in the caller's
// stream and that the caller's stream waits for before the call's results are used.  The Q kernel is bound by memory
// bandwidth, the K and V chains by the latency of their small launches, so together they take about as long as the Q
// kernel alone.  partial_k and partial_v must be different buffers.
extern "C" int tri_write_kv(const void* q, const void* k, const void* v, int batch, int heads_q, int heads_kv, int tokens,
    int64_t q_stride_b, int64_t q_stride_h, int64_t q_stride_t, int64_t k_stride_b, int64_t k_stride_h, int64_t k_stride_t,
    int64_t v_stride_b, int64_t v_stride_h, int64_t v_stride_t, void* q8, float* qa, void* k8, float* ka, float* partial_k,
    float* kstat, void* q4x, float* qa4, void* k4x, void* k4, float* ka4, const int32_t* q_modes, float* partial_v, float* vstat,
    void* v16, void* v8, void* v4, void* v8h, const int32_t* raw_heads, void* stream) {
  const QkArgs a{q, k, batch, heads_q, heads_kv, tokens, q_stride_b, q_stride_h, q_stride_t, k_stride_b, k_stride_h, k_stride_t,
                 q8, qa, k8, ka, partial_k, kstat, q4x, qa4, k4x, k4, ka4, q_modes};
  const VArgs b{v, batch, heads_kv, tokens, v_stride_b, v_stride_h, v_stride_t, partial_v, vstat, v16, v8, v4, v8h, raw_heads};
  if (const int rc = check_qk(a)) return rc;
  if (const int rc = check_v(b)) return rc;
  TRI_CHECK(partial_k != partial_v, "write_kv: the K and V statistics need scratch buffers of their own");
  int device = -1;
  TRI_CUDA(cudaGetDevice(&device), "write_kv");
  TRI_CHECK(device >= 0 && device < TriPerDevice::MaxDevices, "write_kv: device ordinal");
  WriteLanes& lanes = g_lanes[device];
  std::lock_guard<std::mutex> guard(lanes.lock);
  if (!lanes.ready) {
    int least = 0, greatest = 0;
    TRI_CUDA(cudaDeviceGetStreamPriorityRange(&least, &greatest), "write_kv: stream priorities");
    for (int i = 0; i < 2; ++i) {
      // highest priority: the small kernels of the K and V chains get the SM slots that the Q kernel's CTAs free first
      TRI_CUDA(cudaStreamCreateWithPriority(&lanes.side[i], cudaStreamNonBlocking, greatest), "write_kv: side stream");
      TRI_CUDA(cudaEventCreateWithFlags(&lanes.join[i], cudaEventDisableTiming), "write_kv: event");
    }
    TRI_CUDA(cudaEventCreateWithFlags(&lanes.fork, cudaEventDisableTiming), "write_kv: event");
    lanes.ready = true;
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  TRI_CUDA(cudaEventRecord(lanes.fork, s), "write_kv: fork");
  TRI_CUDA(cudaStreamWaitEvent(lanes.side[0], lanes.fork, 0), "write_kv: fork");
  TRI_CUDA(cudaStreamWaitEvent(lanes.side[1], lanes.fork, 0), "write_kv: fork");
  launch_k(a, lanes.side[0]);
  launch_v(b, lanes.side[1]);
  launch_q(a, s);
  TRI_CUDA(cudaEventRecord(lanes.join[0], lanes.side[0]), "write_kv: join");
  TRI_CUDA(cudaEventRecord(lanes.join[1], lanes.side[1]), "write_kv: join");
  TRI_CUDA(cudaStreamWaitEvent(s, lanes.join[0], 0), "write_kv: join");
  TRI_CUDA(cudaStreamWaitEvent(s, lanes.join[1], 0), "write_kv: join");
  return tri_launch_status("write_kv");
}

// Quantise K and V rows with statistics that already exist (the prompt's): the cache write for keys that arrive
// after the prompt.  The same two kernels as above; no statistics pass, INT8 blobs only.
extern "C" int tri_requantize_kv(const void* k, const void* v, int batch, int heads_kv, int tokens, int64_t k_stride_b,
    int64_t k_stride_h, int64_t k_stride_t, int64_t v_stride_b, int64_t v_stride_h, int64_t v_stride_t, const float* kstat,
    const float* vstat, void* k8, float* ka, void* v8, void* stream) {
  TRI_CHECK(k && v && kstat && vstat && k8 && ka && v8, "requantize_kv: null buffers");
  TRI_CHECK(batch > 0 && heads_kv > 0 && tokens > 0 && (tokens + BN - 1) / BN <= MaxTiles, "requantize_kv: bad geometry");
  TRI_CHECK(aligned16(k) && aligned16(v) && k_stride_b % 8 == 0 && k_stride_h % 8 == 0 && k_stride_t % 8 == 0 &&
            v_stride_b % 8 == 0 && v_stride_h % 8 == 0 && v_stride_t % 8 == 0 && aligned16(k8) && aligned16(v8) &&
            aligned16(kstat) && aligned16(vstat), "requantize_kv: BF16 K/V [B,Hkv,T,128], 16-byte aligned rows and blobs");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int tiles = (tokens + BN - 1) / BN, uk = batch * heads_kv;
  launch_chained(quantize_k_kernel, dim3(tiles, uk), dim3(128), 0, s, static_cast<const __nv_bfloat16*>(k), kstat,
      static_cast<uint8_t*>(k8), ka, static_cast<uint8_t*>(nullptr), static_cast<uint8_t*>(nullptr),
      static_cast<float*>(nullptr), tokens, heads_kv, k_stride_b, k_stride_h, k_stride_t);
  launch_chained(pack_v_kernel, dim3(tiles, uk), dim3(256), 0, s, static_cast<const __nv_bfloat16*>(v), vstat,
      static_cast<uint8_t*>(nullptr), static_cast<uint8_t*>(v8), static_cast<uint8_t*>(nullptr), static_cast<uint8_t*>(nullptr),
      tokens, heads_kv, v_stride_b, v_stride_h, v_stride_t, static_cast<const int32_t*>(nullptr));
  return tri_launch_status("requantize_kv");
}
