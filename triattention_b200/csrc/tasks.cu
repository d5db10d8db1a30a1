// Task-table mode of the prefill attention (triattention/kernels/cuda/prefill_sm80.cu:287-292,478-481 of the
// reference): every (Q head, query block) comes with four explicit tile lists instead of a band,
//   pass 0  INT8 scores, fp16 weights,  V' as fp16      pass 2  INT8 scores, 4-bit P codes, INT4 V codes
//   pass 1  INT8 scores, 8-bit P codes, INT8 V codes    pass 3  INT4 scores, 8-bit P codes, INT8 V codes
// groups int32 [Hq*rows*4 + 1] are offsets into entries int32 [...] (tile numbers); block (h, qb) owns
// groups[(h*rows+qb)*4 .. +4].  In a pass only the LAST tile is masked (causal + length), and only if it is the
// block's diagonal tile.  The reference has no caller for this mode (its executor always passes a band table), so
// this is a plain CUDA-core kernel (dp4a) that keeps the interface alive with the reference's arithmetic: one CTA
// per block, four threads per query row (one per 16-key scale group for the scores, one per 32 channels for the
// output).  The banded path, which every caller uses, is the tensor-core kernel in prefill_kernel.cuh.
#include <climits>

#include "abi_internal.h"
#include "common.cuh"

namespace tri {


__device__ __forceinline__ int dp4a_ss(uint32_t a, uint32_t b, int c) {
  int d;
  asm("dp4a.s32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}
__device__ __forceinline__ int dp4a_us(uint32_t a, uint32_t b, int c) {
  int d;
  asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}
// four 4-bit two's-complement values (one per byte, upper nibbles clear) -> four int8
__device__ __forceinline__ uint32_t nibbles_to_s8(uint32_t x) { return __vsub4(x ^ 0x08080808u, 0x08080808u); }

template <typename Out>
__global__ void __launch_bounds__(256) task_kernel(const int32_t* groups, const int32_t* entries, const uint8_t* v16,
    const uint8_t* v8, const uint8_t* v4, const float* vstat, const int8_t* q8, const uint8_t* k8, const float* qa8,
    const float* ka8, const int8_t* q4x, const uint8_t* k4x, const float* qa4, const float* ka4, Out* out, int64_t osb,
    int64_t osh, int64_t ost, int heads_q, int heads_kv, int tokens, float sm_log2, int* err) {
  __shared__ __align__(16) uint8_t ks[K8Bytes];
  __shared__ __align__(16) uint8_t vs[V16Bytes];
  __shared__ __align__(16) uint8_t ps[BM * BN * 2];   // this tile's P: fp16 weights or byte codes, [row][key]
  const int tid = threadIdx.x, row = tid / 4, qd = tid % 4;
  const int qb = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int tiles = (tokens + BN - 1) / BN, qi = qb * BM + row;
  const int64_t qunit = (int64_t)b * heads_q + h, kvunit = (int64_t)b * heads_kv + h / (heads_q / heads_kv);
  const bool row_live = qi < tokens;
  const int32_t* g = groups + ((int64_t)h * tiles + qb) * 4;

  float acc_out[32];
#pragma unroll
  for (int j = 0; j < 32; ++j) acc_out[j] = 0.f;
  float m = -FLT_MAX, denom = 0.f;   // denom: this thread's share (its 16 keys of every tile)
  uint32_t qw[32];

  for (int pass = 0; pass < 4; ++pass) {
    const int begin = g[pass], end = g[pass + 1];
    if (begin >= end) continue;
    const bool q4pass = pass == 3;
    if (q4pass && q4x == nullptr) continue;
    {
      const int8_t* qsrc = (q4pass ? q4x : q8) + (qunit * tokens + qi) * D;
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        const uint4 w = row_live ? reinterpret_cast<const uint4*>(qsrc)[c] : make_uint4(0, 0, 0, 0);
        qw[4 * c] = w.x; qw[4 * c + 1] = w.y; qw[4 * c + 2] = w.z; qw[4 * c + 3] = w.w;
      }
    }
    const float qs = row_live ? (q4pass ? qa4 : qa8)[qunit * tokens + qi] * sm_log2 : FLT_MIN;
    const uint8_t* kblob = q4pass ? k4x : k8;
    const float* kscale = q4pass ? ka4 : ka8;
    const uint8_t* vblob = pass == 0 ? v16 : pass == 2 ? v4 : v8;
    const int vbytes = pass == 0 ? V16Bytes : pass == 2 ? V4Bytes : V8Bytes;

    for (int e = begin; e < end; ++e) {
      const int tile = entries[e];
      if (tile < 0 || tile >= tiles) {          // uniform for the CTA
        if (tid == 0) atomicCAS(err, ErrNone, ErrBadTask);
        continue;
      }
      const bool masked = e == end - 1 && tile == qb;
      const int64_t ht = kvunit * tiles + tile;
      __syncthreads();                          // everyone is done with the previous tile
      for (int i = tid; i < K8Bytes / 16; i += 256)
        reinterpret_cast<uint4*>(ks)[i] = reinterpret_cast<const uint4*>(kblob + ht * K8Bytes)[i];
      for (int i = tid; i < vbytes / 16; i += 256)
        reinterpret_cast<uint4*>(vs)[i] = reinterpret_cast<const uint4*>(vblob + ht * vbytes)[i];
      __syncthreads();

      // ---- scores of this row against the 16 keys of scale group qd (prefill_sm80.cu:158-232) ----
      int acc[16];
      unsigned live = 0xffffu;
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        const int r = qd * 16 + j;
        int a = 0;
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          const uint4 kw = reinterpret_cast<const uint4*>(ks)[(r / 8) * 64 + c * 8 + (r % 8)];
          a = dp4a_ss(qw[4 * c], kw.x, a); a = dp4a_ss(qw[4 * c + 1], kw.y, a);
          a = dp4a_ss(qw[4 * c + 2], kw.z, a); a = dp4a_ss(qw[4 * c + 3], kw.w, a);
        }
        acc[j] = a;
        const int key = tile * BN + r;
        if (masked && (key >= tokens || key > qi || !row_live)) live &= ~(1u << j);
      }
      const float4 k4s = *reinterpret_cast<const float4*>(kscale + ht * 4);
      const float ksc = qd == 0 ? k4s.x : qd == 1 ? k4s.y : qd == 2 ? k4s.z : k4s.w;
      const float slope = qs * ksc;
      // scaled row maximum (prefill_sm80.cu:244-253) and the running maximum
      int amax = INT_MIN;
#pragma unroll
      for (int j = 0; j < 16; ++j) if ((live >> j) & 1u) amax = max(amax, acc[j]);
      float tile_max = live ? slope * (float)amax : -CUDART_INF_F;
      tile_max = fmaxf(tile_max, __shfl_xor_sync(0xffffffffu, tile_max, 1));
      tile_max = fmaxf(tile_max, __shfl_xor_sync(0xffffffffu, tile_max, 2));
      const float n = fmaxf(m, tile_max);
      const float alpha = exp2f(m - n);
      m = n;
      denom *= alpha;
#pragma unroll
      for (int j = 0; j < 32; ++j) acc_out[j] *= alpha;

      if (pass == 0) {
        // ---- fp16 weights against V' in fp16 (prefill_sm80.cu:356-379) ----
        const float off = fmaf(-slope, 12582912.f, -m);
        __half p[16];
        float sum = 0.f;
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const float e = ((live >> j) & 1u) ? exp2f(fmaf(slope, (float)acc[j] + 12582912.f, off)) : 0.f;
          p[j] = __float2half_rn(e);
          sum += __half2float(p[j]);
        }
        denom += sum;
        __half* prow = reinterpret_cast<__half*>(ps) + row * BN;
#pragma unroll
        for (int j = 0; j < 16; ++j) prow[qd * 16 + j] = p[j];
        __syncwarp();                                   // the four threads of a row sit in one warp
        const __half* vh = reinterpret_cast<const __half*>(vs);
        for (int key = 0; key < BN; ++key) {
          const float w = __half2float(prow[key]);
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const int ch = qd * 32 + j;
            acc_out[j] = fmaf(w, __half2float(vh[((ch / 8) * 8 + key / 8) * 64 + (ch % 8) * 8 + key % 8]), acc_out[j]);
          }
        }
      } else {
        // ---- P codes relative to the tile's own base (prefill_sm80.cu:381-441) ----
        const float levels = pass == 2 ? 15.f : 255.f;
        const float ks_max = fmaxf(fmaxf(k4s.x, k4s.y), fmaxf(k4s.z, k4s.w));
        float base = tile_max > -CUDART_INF_F ? tile_max : m;
        base += tile_base_margin(qs * ks_max, base);
        const float bq = exp2f(base - m) / levels;
        const float off = q4pass ? -base : fmaf(-slope, 12582912.f, -base);
        uint32_t code_words[4] = {0u, 0u, 0u, 0u};
        int rs = 0;
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const float sc = q4pass ? (float)acc[j] : (float)acc[j] + 12582912.f;
          const float e = ((live >> j) & 1u) ? exp2f(fmaf(slope, sc, off)) : 0.f;
          const uint32_t code = (__float_as_uint(fmaf(e, levels, PMagicHalf)) >> 8) & 0xffu;   // floor(e * levels + 0.5)
          rs += (int)code;
          code_words[j / 4] |= code << (8 * (j % 4));
        }
        denom = fmaf((float)rs, bq, denom);
        uint4* prow = reinterpret_cast<uint4*>(ps + row * BN);
        prow[qd] = make_uint4(code_words[0], code_words[1], code_words[2], code_words[3]);
        __syncwarp();
        // the row's 64 codes, regrouped like the V blobs: word [blk][s] = keys 16 blk + {2s, 2s+1, 2s+8, 2s+9}
        uint32_t pw[4][4];
#pragma unroll
        for (int blk = 0; blk < 4; ++blk) {
          const uint4 nat = prow[blk];
          pw[blk][0] = __byte_perm(nat.x, nat.z, 0x5410); pw[blk][1] = __byte_perm(nat.x, nat.z, 0x7632);
          pw[blk][2] = __byte_perm(nat.y, nat.w, 0x5410); pw[blk][3] = __byte_perm(nat.y, nat.w, 0x7632);
        }
        const float restore = pass == 2 ? bq * (127.f / 7.f) : bq;
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          const int ch = qd * 32 + j;
          int d = 0;
          if (pass == 2) {
#pragma unroll
            for (int kc = 0; kc < 2; ++kc) {
              const uint4 v = reinterpret_cast<const uint4*>(vs)[((ch / 8) * 2 + kc) * 8 + ch % 8];
              const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
              for (int s = 0; s < 4; ++s) {
                d = dp4a_us(pw[2 * kc][s], nibbles_to_s8(w[s] & 0x0f0f0f0fu), d);
                d = dp4a_us(pw[2 * kc + 1][s], nibbles_to_s8((w[s] >> 4) & 0x0f0f0f0fu), d);
              }
            }
          } else {
#pragma unroll
            for (int blk = 0; blk < 4; ++blk) {
              const uint4 v = reinterpret_cast<const uint4*>(vs)[((ch / 8) * 4 + blk) * 8 + ch % 8];
              d = dp4a_us(pw[blk][0], v.x, d); d = dp4a_us(pw[blk][1], v.y, d);
              d = dp4a_us(pw[blk][2], v.z, d); d = dp4a_us(pw[blk][3], v.w, d);
            }
          }
          acc_out[j] = fmaf((float)d, restore, acc_out[j]);
        }
      }
    }
  }

  // ---- O / denominator, de-normalised (prefill_sm80.cu:466-487) ----
  float total = denom;
  total += __shfl_xor_sync(0xffffffffu, total, 1);
  total += __shfl_xor_sync(0xffffffffu, total, 2);
  if (!row_live) return;
  const float inv = total > 0.f ? 1.f / total : 0.f;
  const float* mean = vstat + kvunit * StatFloats + qd * 32;
  const float* scale = mean + D;
  Out* dst = out + b * osb + h * osh + (int64_t)qi * ost + qd * 32;
#pragma unroll
  for (int j = 0; j < 32; j += 2) {
    Out pair[2] = {static_cast<Out>(fmaf(acc_out[j] * inv, scale[j], mean[j])),
                   static_cast<Out>(fmaf(acc_out[j + 1] * inv, scale[j + 1], mean[j + 1]))};
    *reinterpret_cast<uint32_t*>(dst + j) = *reinterpret_cast<const uint32_t*>(pair);
  }
}

}  // namespace tri

using namespace tri;

extern "C" int tri_attention_tasks(const int32_t* groups, const int32_t* entries, const void* v16, const void* v8,
    const void* v4, const float* vstat, const void* q8, const void* k8, const float* qa8, const float* ka8, const void* q4x,
    const void* k4x, const float* qa4, const float* ka4, void* out, int out_is_half, int64_t out_stride_b,
    int64_t out_stride_h, int64_t out_stride_t, int batch, int heads_q, int heads_kv, int tokens, double scale,
    int* device_error, void* stream) {
  TRI_CHECK(groups && entries && vstat && q8 && k8 && qa8 && ka8 && out && device_error, "attention_tasks: null operands");
  TRI_CHECK(v16 && v8 && v4, "attention_tasks: the task table may name any pass, so V16, V8 and V4 are all needed");
  TRI_CHECK(batch > 0 && heads_q > 0 && heads_kv > 0 && heads_q % heads_kv == 0 && tokens > 0, "attention_tasks: bad geometry");
  TRI_CHECK((tokens + BN - 1) / BN <= MaxTiles, "at most 131072 tokens");
  const bool int4 = q4x != nullptr;
  TRI_CHECK(int4 == (k4x != nullptr) && int4 == (qa4 != nullptr) && int4 == (ka4 != nullptr), "INT4 Q/K operands (all or none)");
  TRI_CHECK(aligned16(out) && out_stride_t % 8 == 0 && out_stride_h % 8 == 0 && out_stride_b % 8 == 0,
            "output [B,Hq,T,128] aligned");
  TRI_CHECK(aligned16(q8) && aligned16(q4x) && aligned16(k8) && aligned16(k4x) && aligned16(v16) && aligned16(v8) &&
            aligned16(v4) && aligned16(ka8) && aligned16(ka4), "attention_tasks: operands must be 16-byte aligned");
  const dim3 grid((tokens + BM - 1) / BM, heads_q, batch);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const float sm_log2 = (float)(scale * 1.4426950408889634);
#define TRI_LAUNCH(T)                                                                                                        \
  task_kernel<T><<<grid, 256, 0, s>>>(groups, entries, static_cast<const uint8_t*>(v16), static_cast<const uint8_t*>(v8),    \
      static_cast<const uint8_t*>(v4), vstat, static_cast<const int8_t*>(q8), static_cast<const uint8_t*>(k8), qa8, ka8,     \
      static_cast<const int8_t*>(q4x), static_cast<const uint8_t*>(k4x), qa4, ka4, static_cast<T*>(out), out_stride_b,       \
      out_stride_h, out_stride_t, heads_q, heads_kv, tokens, sm_log2, device_error)
  if (out_is_half) TRI_LAUNCH(__half); else TRI_LAUNCH(__nv_bfloat16);
#undef TRI_LAUNCH
  return tri_launch_status("attention_tasks");
}
