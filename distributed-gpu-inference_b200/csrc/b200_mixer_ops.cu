// Sequence mixers and feed-forward pieces for decoder designs that keep an fp32 residual stream and run ragged
// batches (prompt portions beside single decoded tokens, packed token-major):
//
//   offset RMS norm            y = x * rsqrt(mean(x^2) + eps) * (1 + w)            fp32 in, storage dtype out
//   post-norm residual update  x += m * norm(y; w_post), optionally followed by the next sublayer's input norm
//   value prep + paged append  per-head unit-RMS values, optional mix with an earlier layer's values, K/V scatter
//                              into pools whose K and V rows have different widths
//   biased paged attention     causal softmax attention of packed query rows over the paged cache with a learned
//                              bias per (distance bucket, head), a per-position query temperature and a per-head
//                              sigmoid output gate
//   gated linear recurrence    S_t = diag(f_t) S_(t-1) + (1 - f_t) v_t^T, o_t = S_t^T q_t with the state in fp32,
//                              carried per sequence in a slot pool; then a per-head weighted RMS norm
//   PolyNorm activation        a N(z) + b N(z^2) + c N(z^3) + e over a token's feed-forward row
//   sigmoid top-k routing, input-scaled expert rows, clamped GLU, combine
//
// Every constant of a design (eps, multipliers, temperatures, limits, table sizes) is a parameter.  Scores, softmax,
// norms, gates of the recurrence, the state and the residual are fp32 whatever the storage dtype T is.  Summation
// orders depend only on a token's own position and sizes, never on how a batch was cut, so a position's result does
// not change with its neighbours in the batch.
#include <algorithm>
#include <type_traits>

#include "../../include/b200_mixers.h"
#include "b200_common.cuh"

namespace b200 {

// this file is a shared library of its own: it carries its own error buffer
char* last_error_buf() {
  static thread_local char buf[kErrBufLen] = {0};
  return buf;
}

namespace {

template <typename F>
int mixer_by_dtype(int dtype, const char* name, F&& f) {
  switch (dtype) {
    case B200_DTYPE_F16:
      return f(static_cast<__half*>(nullptr));
    case B200_DTYPE_BF16:
      return f(static_cast<__nv_bfloat16*>(nullptr));
    case B200_DTYPE_F32:
      return f(static_cast<float*>(nullptr));
    default:
      return fail(B200_EINVAL, "%s: unsupported dtype %d", name, dtype);
  }
}

__device__ __forceinline__ float block_sum_256(float v, float* red) {
  // every thread returns the total; `red` holds 32 floats and may be reused after the call's second barrier
  v = warp_sum(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = (lane < nw) ? red[lane] : 0.f;
  return warp_sum(t);
}

__device__ __forceinline__ float sigmoidf_(float z) { return 1.0f / (1.0f + expf(-z)); }

// ---- offset RMS norm ------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256)
offset_rmsnorm_kernel(T* __restrict__ out, const float* __restrict__ x, const T* __restrict__ w, float eps, int width) {
  __shared__ float red[32];
  const float* xr = x + static_cast<int64_t>(blockIdx.x) * width;
  float ss = 0.f;
  for (int i = threadIdx.x; i < width; i += blockDim.x) ss = fmaf(xr[i], xr[i], ss);
  const float inv = rsqrtf(block_sum_256(ss, red) / static_cast<float>(width) + eps);
  T* orow = out + static_cast<int64_t>(blockIdx.x) * width;
  for (int i = threadIdx.x; i < width; i += blockDim.x)
    orow[i] = Cvt<T>::from_f32(xr[i] * inv * (1.0f + Cvt<T>::to_f32(w[i])));
}

// ---- x += mult * norm(y; w_post); optionally out_next = norm(x; w_next) ------------------------------------------
// One CTA per token.  The updated row is kept in shared memory between the update and the second norm.
template <typename T, typename Y>
__global__ void __launch_bounds__(256)
postnorm_residual_kernel(float* __restrict__ x, const Y* __restrict__ y, int64_t y_stride, const T* __restrict__ w_post,
                         float mult, const T* __restrict__ w_next, T* __restrict__ out_next, float eps, int width) {
  extern __shared__ float row_s[];
  __shared__ float red[32];
  const Y* yr = y + static_cast<int64_t>(blockIdx.x) * y_stride;
  float* xr = x + static_cast<int64_t>(blockIdx.x) * width;
  float ss = 0.f;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    const float v = Cvt<Y>::to_f32(yr[i]);
    ss = fmaf(v, v, ss);
  }
  const float inv = rsqrtf(block_sum_256(ss, red) / static_cast<float>(width) + eps);
  float sx = 0.f;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    const float n = Cvt<Y>::to_f32(yr[i]) * inv * (1.0f + Cvt<T>::to_f32(w_post[i]));
    const float v = xr[i] + mult * n;
    xr[i] = v;
    row_s[i] = v;
    sx = fmaf(v, v, sx);
  }
  if (w_next == nullptr) return;
  const float inv2 = rsqrtf(block_sum_256(sx, red) / static_cast<float>(width) + eps);
  T* orow = out_next + static_cast<int64_t>(blockIdx.x) * width;
  for (int i = threadIdx.x; i < width; i += blockDim.x)
    orow[i] = Cvt<T>::from_f32(row_s[i] * inv2 * (1.0f + Cvt<T>::to_f32(w_next[i])));
}

// ---- value prep + K/V append ------------------------------------------------------------------------------------
// One CTA per token, one warp per kv head (looping).  v <- v / rms(v) per head; with `v_prev` the stored value is
// (1 - lam) v + lam v_prev.  The stored value also goes to `v_keep` (for later layers of the same step) when given.
template <typename T>
__global__ void __launch_bounds__(128)
value_prep_append_kernel(const T* __restrict__ k, int64_t k_stride, const T* __restrict__ v, int64_t v_stride,
                         const T* __restrict__ v_prev, T* __restrict__ v_keep, float lam, float eps,
                         T* __restrict__ k_pool, T* __restrict__ v_pool, const int64_t* __restrict__ slot_mapping,
                         int G, int dk, int dv, int block_size, int64_t max_blocks) {
  const int tok = blockIdx.x;
  const int64_t slot = slot_mapping[tok];
  const int64_t blk = slot >= 0 ? slot / block_size : -1;
  const bool store = blk >= 0 && blk < max_blocks;
  const int off = store ? static_cast<int>(slot - blk * block_size) : 0;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  for (int g = warp; g < G; g += nw) {
    const T* vr = v + tok * v_stride + g * dv;
    float ss = 0.f;
    for (int c = lane; c < dv; c += 32) {
      const float f = Cvt<T>::to_f32(vr[c]);
      ss = fmaf(f, f, ss);
    }
    const float inv = rsqrtf(warp_sum(ss) / static_cast<float>(dv) + eps);
    T* dst = store ? v_pool + ((blk * G + g) * block_size + off) * dv : nullptr;
    for (int c = lane; c < dv; c += 32) {
      float f = Cvt<T>::to_f32(vr[c]) * inv;
      if (v_prev) f = (1.0f - lam) * f + lam * Cvt<T>::to_f32(v_prev[static_cast<int64_t>(tok) * G * dv + g * dv + c]);
      const T r = Cvt<T>::from_f32(f);
      if (dst) dst[c] = r;
      if (v_keep) v_keep[static_cast<int64_t>(tok) * G * dv + g * dv + c] = r;
    }
  }
  if (store) {
    for (int i = threadIdx.x; i < G * dk; i += blockDim.x) {
      const int g = i / dk, d = i - g * dk;
      k_pool[((blk * G + g) * block_size + off) * dk + d] = k[tok * k_stride + i];
    }
  }
}

// ---- biased paged attention over packed query rows ----------------------------------------------------------------
// A CTA serves up to QT consecutive tokens of ONE sequence and one kv head: QT * (H / G) query rows.  Keys are
// walked in tiles of 32 from position 0 (tile borders are fixed in the sequence, so the online-softmax order of a
// position does not depend on how the prompt was cut).  K and V tiles sit in shared memory as fp32; a warp owns RW
// rows, lane j scores key j of the tile, then the lanes split the value columns.
struct AttnTile {
  int tok0;   // first packed row of the tile
  int count;  // tokens in the tile (<= QT)
  int seq;    // row of the block table
};

constexpr int kAttnWarps = 8;
constexpr int kKeyTile = 32;

template <typename T, int RW, int DVL, int NCH>
__global__ void __launch_bounds__(kAttnWarps * 32)
biased_paged_attn_kernel(T* __restrict__ out, const T* __restrict__ q, int64_t q_stride, const T* __restrict__ gate,
                         int64_t gate_stride, const T* __restrict__ k_pool, const T* __restrict__ v_pool,
                         const int32_t* __restrict__ block_tables, int table_stride, const AttnTile* __restrict__ tiles,
                         const int32_t* __restrict__ tok_pos, const float* __restrict__ bias_lut, int lut_len,
                         float scale, float temp_coef, int temp_every, int H, int G, int dk, int dv, int block_size) {
  // NCH > 0: K / V rows are fetched as 16-byte chunks, NCH per thread, into registers one key tile AHEAD of the
  // tile being computed (needs dk and dv to be multiples of 16 bytes).  NCH == 0: element-wise loads, any sizes.
  extern __shared__ __align__(16) float smem[];
  const int dkp = (dk + 3) & ~3;            // padded row length of K / q rows (multiple of 4 floats)
  const int ks = dkp + 4;                   // K row stride: 16-byte aligned and conflict-free for 128-bit reads
  const int rep = H / G;
  const AttnTile tile = tiles[blockIdx.x];
  const int g = blockIdx.y;
  const int n_rows = tile.count * rep;
  float* k_s = smem;                        // [32][ks]
  float* v_s = k_s + kKeyTile * ks;         // [32][dv]
  float* q_s = v_s + kKeyTile * dv;         // [rows][dkp]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  // query rows -> shared memory (fp32, zero padded)
  for (int i = threadIdx.x; i < kAttnWarps * RW * dkp; i += blockDim.x) {
    const int r = i / dkp, d = i - r * dkp;
    const int t = r / rep, hh = g * rep + (r - t * rep);
    q_s[i] = (r < n_rows && d < dk) ? Cvt<T>::to_f32(q[(tile.tok0 + t) * q_stride + hh * dk + d]) : 0.f;
  }
  const int pos_last = tok_pos[tile.tok0 + tile.count - 1];
  const int32_t* table = block_tables + static_cast<int64_t>(tile.seq) * table_stride;

  // per-row state of this warp's rows
  float m[RW], l[RW], acc[RW][DVL], qmul[RW];
  int pos[RW], head[RW];
  bool live[RW];
#pragma unroll
  for (int r = 0; r < RW; ++r) {
    const int row = warp * RW + r;
    live[r] = row < n_rows;
    const int t = live[r] ? row / rep : 0;
    head[r] = g * rep + (live[r] ? row - t * rep : 0);
    pos[r] = live[r] ? tok_pos[tile.tok0 + t] : -1;
    const float steps = static_cast<float>((pos[r] + 1) / max(temp_every, 1));
    qmul[r] = scale * (1.0f + temp_coef * logf(steps + 1.0f));
    m[r] = -INFINITY;
    l[r] = 0.f;
#pragma unroll
    for (int c = 0; c < DVL; ++c) acc[r][c] = 0.f;
  }

  constexpr int VN = 16 / sizeof(T);
  constexpr int NR = NCH > 0 ? NCH : 1;
  const int kc = dk / VN, vc = dv / VN;               // chunks per K / V row
  const int n_chunks = kKeyTile * (kc + vc);
  int4 regs[NR];
  const int bs_shift = (block_size & (block_size - 1)) == 0 ? __ffs(block_size) - 1 : -1;
  // the chunks a thread moves are the same for every key tile: (is V, key within the tile, first element) once
  int ch_j[NR], ch_e[NR];
  bool ch_v[NR], ch_ok[NR];
#pragma unroll
  for (int u = 0; u < NR; ++u) {
    const int c = threadIdx.x + u * kAttnWarps * 32;
    ch_ok[u] = NCH > 0 && c < n_chunks;
    ch_v[u] = c >= kKeyTile * kc;
    const int cc = ch_v[u] ? c - kKeyTile * kc : c;
    const int per = max(ch_v[u] ? vc : kc, 1);
    ch_j[u] = cc / per;
    ch_e[u] = (cc - ch_j[u] * per) * VN;
  }
  auto prefetch = [&](int j0) {
    const int n_keys = min(kKeyTile, pos_last + 1 - j0);
#pragma unroll
    for (int u = 0; u < NR; ++u) {
      regs[u] = make_int4(0, 0, 0, 0);
      if (ch_ok[u] && ch_j[u] < n_keys) {
        const int key = j0 + ch_j[u];
        const int bi = bs_shift >= 0 ? key >> bs_shift : key / block_size;   // pages are a power of two as a rule
        const int64_t row = (static_cast<int64_t>(table[bi]) * G + g) * block_size + (key - bi * block_size);
        regs[u] = *reinterpret_cast<const int4*>(ch_v[u] ? v_pool + row * dv + ch_e[u] : k_pool + row * dk + ch_e[u]);
      }
    }
  };
  auto commit = [&]() {
#pragma unroll
    for (int u = 0; u < NR; ++u) {
      if (ch_ok[u]) {
        const T* el = reinterpret_cast<const T*>(&regs[u]);
        float* dst = ch_v[u] ? v_s + ch_j[u] * dv + ch_e[u] : k_s + ch_j[u] * ks + ch_e[u];
        if constexpr (VN == 8) {
          *reinterpret_cast<float4*>(dst) = make_float4(Cvt<T>::to_f32(el[0]), Cvt<T>::to_f32(el[1]), Cvt<T>::to_f32(el[2]), Cvt<T>::to_f32(el[3]));
          *reinterpret_cast<float4*>(dst + 4) = make_float4(Cvt<T>::to_f32(el[4]), Cvt<T>::to_f32(el[5]), Cvt<T>::to_f32(el[6]), Cvt<T>::to_f32(el[7]));
        } else {
          *reinterpret_cast<float4*>(dst) = make_float4(Cvt<T>::to_f32(el[0]), Cvt<T>::to_f32(el[1]), Cvt<T>::to_f32(el[2]), Cvt<T>::to_f32(el[3]));
        }
      }
    }
  };
  if constexpr (NCH > 0) prefetch(0);

  for (int j0 = 0; j0 <= pos_last; j0 += kKeyTile) {
    __syncthreads();  // previous tile fully consumed (and q_s written, on the first pass)
    const int n_keys = min(kKeyTile, pos_last + 1 - j0);
    if constexpr (NCH > 0) {
      commit();
    } else {
      for (int i = threadIdx.x; i < kKeyTile * dkp; i += blockDim.x) {
        const int j = i / dkp, d = i - j * dkp;
        float f = 0.f;
        if (j < n_keys && d < dk) {
          const int key = j0 + j;
          const int64_t blk = table[key / block_size];
          f = Cvt<T>::to_f32(k_pool[((blk * G + g) * block_size + key % block_size) * dk + d]);
        }
        k_s[j * ks + d] = f;
      }
      for (int i = threadIdx.x; i < kKeyTile * dv; i += blockDim.x) {
        const int j = i / dv, c = i - j * dv;
        float f = 0.f;
        if (j < n_keys) {
          const int key = j0 + j;
          const int64_t blk = table[key / block_size];
          f = Cvt<T>::to_f32(v_pool[((blk * G + g) * block_size + key % block_size) * dv + c]);
        }
        v_s[i] = f;
      }
    }
    __syncthreads();
    if constexpr (NCH > 0) {
      if (j0 + kKeyTile <= pos_last) prefetch(j0 + kKeyTile);
    }

    if (warp * RW < n_rows) {   // warps without a live row only help with the loads and barriers
    // scores: lane = key of the tile
    float s[RW];
#pragma unroll
    for (int r = 0; r < RW; ++r) s[r] = 0.f;
    const float4* kr = reinterpret_cast<const float4*>(k_s + lane * ks);
    for (int d4 = 0; d4 < dkp / 4; ++d4) {
      const float4 kv = kr[d4];
#pragma unroll
      for (int r = 0; r < RW; ++r) {
        const float4 qv = reinterpret_cast<const float4*>(q_s + (warp * RW + r) * dkp)[d4];  // broadcast read
        s[r] = fmaf(qv.x, kv.x, s[r]);
        s[r] = fmaf(qv.y, kv.y, s[r]);
        s[r] = fmaf(qv.z, kv.z, s[r]);
        s[r] = fmaf(qv.w, kv.w, s[r]);
      }
    }
    float p[RW];
#pragma unroll
    for (int r = 0; r < RW; ++r) {
      const int key = j0 + lane;
      const bool seen = live[r] && key <= pos[r];
      const bool any = live[r] && j0 <= pos[r];  // warp-uniform
      float sc = -INFINITY;
      if (seen) {
        const int dist = min(pos[r] - key, lut_len - 1);
        sc = s[r] * qmul[r] + bias_lut[head[r] * lut_len + dist];
      }
      p[r] = 0.f;
      if (any) {
        const float m_new = fmaxf(m[r], warp_max(sc));
        const float corr = expf(m[r] - m_new);
        p[r] = seen ? expf(sc - m_new) : 0.f;
        l[r] = l[r] * corr + warp_sum(p[r]);
        m[r] = m_new;
#pragma unroll
        for (int c = 0; c < DVL; ++c) acc[r][c] *= corr;
      }
    }
    // values: lane = column (plus 32 c)
    for (int j = 0; j < n_keys; ++j) {
      float vv[DVL];
#pragma unroll
      for (int c = 0; c < DVL; ++c) {
        const int col = lane + 32 * c;
        vv[c] = col < dv ? v_s[j * dv + col] : 0.f;
      }
#pragma unroll
      for (int r = 0; r < RW; ++r) {
        const float pj = __shfl_sync(0xffffffffu, p[r], j);
#pragma unroll
        for (int c = 0; c < DVL; ++c) acc[r][c] = fmaf(pj, vv[c], acc[r][c]);
      }
    }
    }
  }

#pragma unroll
  for (int r = 0; r < RW; ++r) {
    if (!live[r]) continue;
    const int row = warp * RW + r;
    const int t = row / rep;
    const int64_t n = tile.tok0 + t;
    const float gt = gate ? sigmoidf_(Cvt<T>::to_f32(gate[n * gate_stride + head[r]])) : 1.0f;
    const float inv = gt / l[r];
#pragma unroll
    for (int c = 0; c < DVL; ++c) {
      const int col = lane + 32 * c;
      if (col < dv) out[(n * H + head[r]) * dv + col] = Cvt<T>::from_f32(acc[r][c] * inv);
    }
  }
}

// ---- biased attention for prompt portions on the tensor cores (16-bit storage types) --------------------------------
// A CTA serves up to 64 consecutive tokens of one sequence and ONE query head; warp w owns rows 16 w .. 16 w + 15.
// Keys are walked in tiles of 64 from position 0.  K and V tiles arrive by cp.async, double buffered, and stay in
// their storage type; S = Q K^T and O += P V are mma.sync m16n8k16 with fp32 accumulators in registers, the softmax
// (scale, temperature, bias, causal mask, running max and sum) runs in fp32 on the S fragments, and only the
// weights P are rounded to the storage type as the left operand of P V.  V fragments come from ldmatrix.trans.
template <typename T>
struct Mma16;
template <>
struct Mma16<__nv_bfloat16> {
  static __device__ __forceinline__ void mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  }
  static __device__ __forceinline__ uint32_t pack(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&v);
  }
};
template <>
struct Mma16<__half> {
  static __device__ __forceinline__ void mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  }
  static __device__ __forceinline__ uint32_t pack(float lo, float hi) {
    const __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&v);
  }
};

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gmem_src, bool valid) {
  const uint32_t dst = static_cast<uint32_t>(__cvta_generic_to_shared(smem_dst));
  const int bytes = valid ? 16 : 0;  // fewer source bytes than 16: the rest is zero-filled
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(gmem_src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

constexpr int kMmaRows = 64;   // query rows per CTA
constexpr int kMmaKeys = 64;   // keys per tile

// KSPLIT (tiles of at most 16 rows, i.e. decoded tokens): all four warps work on the SAME 16 rows and each takes 16
// of a tile's 64 keys; their running (max, sum, output) are merged through shared memory at the end.
template <typename T, int DV8, bool KSPLIT>
__global__ void __launch_bounds__(128)
biased_prompt_attn_mma_kernel(T* __restrict__ out, const T* __restrict__ q, int64_t q_stride, const T* __restrict__ gate,
                              int64_t gate_stride, const T* __restrict__ k_pool, const T* __restrict__ v_pool,
                              const int32_t* __restrict__ block_tables, int table_stride,
                              const AttnTile* __restrict__ tiles, const int32_t* __restrict__ tok_pos,
                              const float* __restrict__ bias_lut, int lut_len, int lut_in_smem, int q_vec, float scale,
                              float temp_coef, int temp_every, int H, int G, int dk, int dv, int block_size) {
  // Row r of the CTA's 64 is (token r / rep, head g * rep + r % rep): the heads of a kv group share the K / V tiles.
  extern __shared__ __align__(16) unsigned char smem_raw[];
  constexpr int dvp = DV8 * 8;
  const int ldq = dk + 8, ldv = dvp + 8;       // element strides: 16-byte multiples, conflict-free fragment reads
  T* q_s = reinterpret_cast<T*>(smem_raw);     // [64][ldq]
  T* k_s = q_s + kMmaRows * ldq;               // 2 x [64][ldq]
  T* v_s = k_s + 2 * kMmaKeys * ldq;           // 2 x [64][ldv]
  float* lut_s = reinterpret_cast<float*>(v_s + 2 * kMmaKeys * ldv);
  const AttnTile tile = tiles[blockIdx.x];
  const int g = blockIdx.y, rep = H / G;
  const int n_rows = tile.count * rep;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int gq = lane >> 2, tq = lane & 3;
  const int pos0 = tok_pos[tile.tok0];
  const int pos_last = pos0 + tile.count - 1;
  const int32_t* table = block_tables + static_cast<int64_t>(tile.seq) * table_stride;
  if (lut_in_smem) {   // the group's heads, one after the other
    for (int i = threadIdx.x; i < rep * lut_len; i += blockDim.x) lut_s[i] = bias_lut[static_cast<int64_t>(g) * rep * lut_len + i];
  }
  const int qc = dk / 8, vc = dvp / 8;          // 16-byte chunks per row

  // Q tile (rows beyond the tile's are zero); element-wise when the rows are not 16-byte aligned
  if (q_vec) {
    for (int c = threadIdx.x; c < kMmaRows * qc; c += blockDim.x) {
      const int r = c / qc, e = (c - r * qc) * 8;
      const bool ok = r < n_rows;
      const int t = r / rep, hh = g * rep + (r - t * rep);
      cp_async16(q_s + r * ldq + e, ok ? q + (tile.tok0 + t) * q_stride + hh * dk + e : q, ok);
    }
  } else {
    for (int i = threadIdx.x; i < kMmaRows * dk; i += blockDim.x) {
      const int r = i / dk, d = i - r * dk;
      const int t = r / rep, hh = g * rep + (r - t * rep);
      q_s[r * ldq + d] = r < n_rows ? q[(tile.tok0 + t) * q_stride + hh * dk + d] : Cvt<T>::from_f32(0.f);
    }
  }
  // a thread always moves the same 16-byte column of the rows j = row0, row0 + step, ...: no division per chunk
  const int bs_shift = (block_size & (block_size - 1)) == 0 ? __ffs(block_size) - 1 : -1;
  const int k_step = blockDim.x / qc, k_row0 = threadIdx.x / qc, k_e = (threadIdx.x - k_row0 * qc) * 8;
  const int v_step = blockDim.x / vc, v_row0 = threadIdx.x / vc, v_e = (threadIdx.x - v_row0 * vc) * 8;
  auto pool_row = [&](int key) -> int64_t {
    const int bi = bs_shift >= 0 ? key >> bs_shift : key / block_size;
    return (static_cast<int64_t>(table[bi]) * G + g) * block_size + (key - bi * block_size);
  };
  auto load_kv = [&](int j0, int stage) {
    T* kd = k_s + stage * kMmaKeys * ldq;
    T* vd = v_s + stage * kMmaKeys * ldv;
    if (k_row0 < k_step) {
      for (int j = k_row0; j < kMmaKeys; j += k_step) {
        const int key = j0 + j;
        const bool ok = key <= pos_last;
        cp_async16(kd + j * ldq + k_e, k_pool + (ok ? pool_row(key) * dk + k_e : 0), ok);
      }
    }
    if (v_row0 < v_step) {
      const bool col_ok = v_e < dv;
      for (int j = v_row0; j < kMmaKeys; j += v_step) {
        const int key = j0 + j;
        const bool ok = col_ok && key <= pos_last;
        cp_async16(vd + j * ldv + v_e, v_pool + (ok ? pool_row(key) * dv + v_e : 0), ok);
      }
    }
  };
  load_kv(0, 0);
  cp_async_commit();

  const int row_a = (KSPLIT ? 0 : warp * 16) + gq;       // this thread's rows: row_a and row_a + 8
  int posr[2], headr[2], tokr[2];
  const float* lut[2];
  float qmul[2], m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int r = row_a + 8 * i;
    tokr[i] = r / rep;
    headr[i] = g * rep + (r - tokr[i] * rep);
    posr[i] = r < n_rows ? pos0 + tokr[i] : -1;
    lut[i] = lut_in_smem ? lut_s + (r - tokr[i] * rep) * lut_len : bias_lut + static_cast<int64_t>(headr[i]) * lut_len;
    const float steps = static_cast<float>((posr[i] + 1) / max(temp_every, 1));
    qmul[i] = scale * (1.0f + temp_coef * logf(steps + 1.0f));
  }
  const int warp_pos_max = KSPLIT ? pos_last : pos0 + min((warp * 16 + 15) / rep, tile.count - 1);
  const bool warp_live = KSPLIT || warp * 16 < n_rows;
  constexpr int NT = KSPLIT ? 2 : 8;                     // 8-key n-tiles of a key tile this warp scores
  const int nt0 = KSPLIT ? 2 * warp : 0;
  float o[DV8][4];
#pragma unroll
  for (int n = 0; n < DV8; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;

  const int n_kt = pos_last / kMmaKeys + 1;
  for (int it = 0; it < n_kt; ++it) {
    if (it + 1 < n_kt) {
      load_kv((it + 1) * kMmaKeys, (it + 1) & 1);
      cp_async_commit();
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    const int j0 = it * kMmaKeys;
    if (warp_live && j0 <= warp_pos_max) {
      const T* kt = k_s + (it & 1) * kMmaKeys * ldq;
      const T* vt = v_s + (it & 1) * kMmaKeys * ldv;
      float s[NT][4];
#pragma unroll
      for (int n = 0; n < NT; ++n) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f;
      for (int kk = 0; kk < dk / 16; ++kk) {
        uint32_t a[4];
        const T* qa = q_s + row_a * ldq + kk * 16 + 2 * tq;
        a[0] = *reinterpret_cast<const uint32_t*>(qa);
        a[1] = *reinterpret_cast<const uint32_t*>(qa + 8 * ldq);
        a[2] = *reinterpret_cast<const uint32_t*>(qa + 8);
        a[3] = *reinterpret_cast<const uint32_t*>(qa + 8 * ldq + 8);
#pragma unroll
        for (int n = 0; n < NT; ++n) {
          const T* kb = kt + ((nt0 + n) * 8 + gq) * ldq + kk * 16 + 2 * tq;
          Mma16<T>::mma(s[n], a, *reinterpret_cast<const uint32_t*>(kb), *reinterpret_cast<const uint32_t*>(kb + 8));
        }
      }
      // fp32 softmax on the fragments: element e of s[n] is (row gq + 8 (e >> 1), key 8 (nt0 + n) + 2 tq + (e & 1))
      float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
      for (int n = 0; n < NT; ++n) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int i = e >> 1;
          const int key = j0 + (nt0 + n) * 8 + 2 * tq + (e & 1);
          float sc = -INFINITY;
          if (key <= posr[i]) sc = s[n][e] * qmul[i] + lut[i][min(posr[i] - key, lut_len - 1)];
          s[n][e] = sc;
          mx[i] = fmaxf(mx[i], sc);
        }
      }
      float corr[2], msafe[2];
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 1));
        mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 2));
        const float m_new = fmaxf(m[i], mx[i]);
        msafe[i] = m_new == -INFINITY ? 0.f : m_new;   // a row that sees no key yet keeps weights 0, not NaN
        corr[i] = expf(m[i] - msafe[i]);
        m[i] = m_new;
      }
      float part[2] = {0.f, 0.f};
#pragma unroll
      for (int n = 0; n < NT; ++n) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float pexp = expf(s[n][e] - msafe[e >> 1]);
          s[n][e] = pexp;
          part[e >> 1] += pexp;
        }
      }
#pragma unroll
      for (int i = 0; i < 2; ++i) l[i] = l[i] * corr[i] + part[i];   // per-thread share of the row sum
#pragma unroll
      for (int n = 0; n < DV8; ++n) {
        o[n][0] *= corr[0];
        o[n][1] *= corr[0];
        o[n][2] *= corr[1];
        o[n][3] *= corr[1];
      }
#pragma unroll
      for (int k2 = 0; k2 < NT / 2; ++k2) {
        uint32_t a[4];
        a[0] = Mma16<T>::pack(s[2 * k2][0], s[2 * k2][1]);
        a[1] = Mma16<T>::pack(s[2 * k2][2], s[2 * k2][3]);
        a[2] = Mma16<T>::pack(s[2 * k2 + 1][0], s[2 * k2 + 1][1]);
        a[3] = Mma16<T>::pack(s[2 * k2 + 1][2], s[2 * k2 + 1][3]);
        const int key16 = (nt0 / 2 + k2) * 16;           // first key (within the tile) of this 16-key step
#pragma unroll
        for (int n = 0; n < DV8; n += 2) {
          const T* vrow = vt + (key16 + (lane & 7) + ((lane >> 3) & 1) * 8) * ldv + n * 8 + (lane >> 4) * 8;
          const uint32_t addr = static_cast<uint32_t>(__cvta_generic_to_shared(vrow));
          uint32_t b0, b1, b2, b3;
          asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                       : "=r"(b0), "=r"(b1), "=r"(b2), "=r"(b3)
                       : "r"(addr));
          Mma16<T>::mma(o[n], a, b0, b1);
          Mma16<T>::mma(o[n + 1], a, b2, b3);
        }
      }
    }
    __syncthreads();   // the stage just read is the target of the load after next
  }
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    l[i] += __shfl_xor_sync(0xffffffffu, l[i], 1);
    l[i] += __shfl_xor_sync(0xffffffffu, l[i], 2);
  }
  if constexpr (KSPLIT) {
    // merge the four warps' partial results for the 16 shared rows: every warp rescales its own to the common
    // maximum and the sums are taken warp 0, 1, 2, 3 in order; the K / V stages are free now
    float* mg = reinterpret_cast<float*>(k_s);            // [4 warps][16 rows] maxima, then [4][16] sums
    float* og = mg + 128;                                  // [4 warps][16 rows][dvp]
    if (tq == 0) {
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        mg[warp * 16 + gq + 8 * i] = m[i];
        mg[64 + warp * 16 + gq + 8 * i] = l[i];
      }
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int r = gq + 8 * i;
      float mall = fmaxf(fmaxf(mg[r], mg[16 + r]), fmaxf(mg[32 + r], mg[48 + r]));
      mall = mall == -INFINITY ? 0.f : mall;
      const float w = expf(m[i] - mall);                  // this warp's weight in the merge
      float lsum = 0.f;
#pragma unroll
      for (int w2 = 0; w2 < 4; ++w2) lsum += mg[64 + w2 * 16 + r] * expf(mg[w2 * 16 + r] - mall);
      l[i] = lsum;
#pragma unroll
      for (int n = 0; n < DV8; ++n) {
        og[(warp * 16 + r) * dvp + n * 8 + 2 * tq] = o[n][2 * i] * w;
        og[(warp * 16 + r) * dvp + n * 8 + 2 * tq + 1] = o[n][2 * i + 1] * w;
      }
    }
    __syncthreads();
    if (warp != 0) return;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int r = gq + 8 * i;
#pragma unroll
      for (int n = 0; n < DV8; ++n) {
        const int c = n * 8 + 2 * tq;
        o[n][2 * i] = (og[r * dvp + c] + og[(16 + r) * dvp + c]) + (og[(32 + r) * dvp + c] + og[(48 + r) * dvp + c]);
        o[n][2 * i + 1] = (og[r * dvp + c + 1] + og[(16 + r) * dvp + c + 1]) + (og[(32 + r) * dvp + c + 1] + og[(48 + r) * dvp + c + 1]);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int r = row_a + 8 * i;
    if (r >= n_rows) continue;
    const int64_t n_tok = tile.tok0 + tokr[i];
    const int h = headr[i];
    const float gt = gate ? sigmoidf_(Cvt<T>::to_f32(gate[n_tok * gate_stride + h])) : 1.0f;
    const float inv = gt / l[i];
    T* orow = out + (n_tok * H + h) * dv;
#pragma unroll
    for (int n = 0; n < DV8; ++n) {
      const int col = n * 8 + 2 * tq;
      if (col < dv) {   // dv is a multiple of 8: col + 1 < dv as well
        orow[col] = Cvt<T>::from_f32(o[n][2 * i] * inv);
        orow[col + 1] = Cvt<T>::from_f32(o[n][2 * i + 1] * inv);
      }
    }
  }
}

// ---- grouped linear for expert-sorted rows (16-bit storage) ---------------------------------------------------------
// out[r] = xs[r] . w[e]^T for the rows offsets[e] <= r < offsets[e + 1]; the offsets stay on the device, so routing
// needs no copy to the host and all experts run in one launch.  CTA = 16 rows x 256 output columns of one expert
// (each of 4 warps: 16 x 64 with mma.sync m16n8k16, fp32 accumulators); K in chunks of 64 by cp.async, two stages.
// CTAs whose row tile lies beyond their expert's rows leave at once.
constexpr int kGrpRows = 16, kGrpCols = 256, kGrpK = 64;

template <typename T>
__global__ void __launch_bounds__(128)
grouped_linear_kernel(T* __restrict__ out, const T* __restrict__ xs, const T* __restrict__ w,
                      const int32_t* __restrict__ offsets, int N, int K) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int e = blockIdx.y;
  const int row0 = offsets[e] + blockIdx.z * kGrpRows;
  const int row_end = offsets[e + 1];
  if (row0 >= row_end) return;
  const int n0 = blockIdx.x * kGrpCols;
  constexpr int ld = kGrpK + 8;
  T* x_s = reinterpret_cast<T*>(smem_raw);            // 2 x [16][ld]
  T* w_s = x_s + 2 * kGrpRows * ld;                   // 2 x [256][ld]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, gq = lane >> 2, tq = lane & 3;
  const T* wbase = w + static_cast<int64_t>(e) * N * K;
  auto load = [&](int kc, int stage) {
    {
      const int r = threadIdx.x >> 3, e8 = (threadIdx.x & 7) * 8;
      const bool ok = row0 + r < row_end && kc + e8 < K;
      cp_async16(x_s + (stage * kGrpRows + r) * ld + e8, ok ? xs + static_cast<int64_t>(row0 + r) * K + kc + e8 : xs, ok);
    }
#pragma unroll 4
    for (int i = 0; i < kGrpCols * 8 / 128; ++i) {
      const int c = threadIdx.x + i * 128;
      const int n = c >> 3, e8 = (c & 7) * 8;
      const bool ok = n0 + n < N && kc + e8 < K;
      cp_async16(w_s + (stage * kGrpCols + n) * ld + e8, ok ? wbase + static_cast<int64_t>(n0 + n) * K + kc + e8 : wbase, ok);
    }
  };
  float acc[8][4];
#pragma unroll
  for (int n = 0; n < 8; ++n) acc[n][0] = acc[n][1] = acc[n][2] = acc[n][3] = 0.f;
  const int n_kc = (K + kGrpK - 1) / kGrpK;
  load(0, 0);
  cp_async_commit();
  for (int it = 0; it < n_kc; ++it) {
    if (it + 1 < n_kc) {
      load((it + 1) * kGrpK, (it + 1) & 1);
      cp_async_commit();
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    const T* xt = x_s + (it & 1) * kGrpRows * ld;
    const T* wt = w_s + ((it & 1) * kGrpCols + warp * 64) * ld;
#pragma unroll
    for (int kk = 0; kk < kGrpK / 16; ++kk) {
      uint32_t a[4];
      const T* xa = xt + gq * ld + kk * 16 + 2 * tq;
      a[0] = *reinterpret_cast<const uint32_t*>(xa);
      a[1] = *reinterpret_cast<const uint32_t*>(xa + 8 * ld);
      a[2] = *reinterpret_cast<const uint32_t*>(xa + 8);
      a[3] = *reinterpret_cast<const uint32_t*>(xa + 8 * ld + 8);
#pragma unroll
      for (int n = 0; n < 8; ++n) {
        const T* wb = wt + (n * 8 + gq) * ld + kk * 16 + 2 * tq;
        Mma16<T>::mma(acc[n], a, *reinterpret_cast<const uint32_t*>(wb), *reinterpret_cast<const uint32_t*>(wb + 8));
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int r = row0 + gq + 8 * i;
    if (r >= row_end) continue;
    T* orow = out + static_cast<int64_t>(r) * N;
#pragma unroll
    for (int n = 0; n < 8; ++n) {
      const int col = n0 + warp * 64 + n * 8 + 2 * tq;
      if (col < N) orow[col] = Cvt<T>::from_f32(acc[n][2 * i]);
      if (col + 1 < N) orow[col + 1] = Cvt<T>::from_f32(acc[n][2 * i + 1]);
    }
  }
}

// ---- gated linear recurrence ------------------------------------------------------------------------------------
// One CTA per (sequence, head).  The state [dk][dv] lives in shared memory for the whole portion; thread (rg, c)
// owns column c and the rows i = rg, rg + RG, ...  Inputs of token t + 1 are fetched while token t is computed.
struct ScanSeq {
  int tok0;   // first packed row
  int count;  // tokens of this sequence in the step
  int slot;   // state slot
  int fresh;  // 1: the sequence starts here, the state is zero
};

constexpr int kScanCols = 32;   // value columns per CTA (fixed, so the row-sum order never depends on the batch)
constexpr int kScanRG = 256 / kScanCols;
constexpr int kScanPF = 4;      // input elements per thread and token: 2 dk + 32 <= 1024

template <typename T>
__global__ void __launch_bounds__(256)
gated_scan_kernel(float* __restrict__ o_raw, const T* __restrict__ zq, const T* __restrict__ zf, const T* __restrict__ v,
                  int64_t in_stride, const T* __restrict__ f_bias, const T* __restrict__ lower, float* __restrict__ state,
                  const ScanSeq* __restrict__ seqs, int H, int dk, int dv) {
  extern __shared__ float smem[];
  const ScanSeq sq = seqs[blockIdx.x];
  const int h = blockIdx.y;
  const int col0 = blockIdx.z * kScanCols;
  const int ncol = min(kScanCols, dv - col0);
  const int c = threadIdx.x % kScanCols, rg = threadIdx.x / kScanCols;
  float* S = smem;                              // [dk][kScanCols]
  float* in_s = S + dk * kScanCols;             // 2 x (q[dk], f[dk], v[kScanCols])
  const int in_len = 2 * dk + kScanCols;
  float* part = in_s + 2 * in_len;              // [kScanRG][kScanCols]
  float* st = state + (static_cast<int64_t>(sq.slot) * H + h) * dk * dv;
  for (int i = threadIdx.x; i < dk * kScanCols; i += blockDim.x) {
    const int r = i / kScanCols, cc = i - r * kScanCols;
    S[i] = (sq.fresh || cc >= ncol) ? 0.f : st[r * dv + col0 + cc];
  }
  // element i of a token's inputs is always handled by thread i % 256: its bias / bound are loaded once
  float bias_r[kScanPF], low_r[kScanPF];
#pragma unroll
  for (int u = 0; u < kScanPF; ++u) {
    const int i = threadIdx.x + u * 256;
    bias_r[u] = low_r[u] = 0.f;
    if (i >= dk && i < 2 * dk) {
      bias_r[u] = Cvt<T>::to_f32(f_bias[h * dk + i - dk]);
      low_r[u] = Cvt<T>::to_f32(lower[h * dk + i - dk]);
    }
  }
  T raw[kScanPF];
  auto fetch = [&](int t) {     // raw loads only: nothing waits for them until `commit`
    const int64_t row = static_cast<int64_t>(sq.tok0 + t) * in_stride;
#pragma unroll
    for (int u = 0; u < kScanPF; ++u) {
      const int i = threadIdx.x + u * 256;
      raw[u] = Cvt<T>::from_f32(0.f);
      if (i < dk) raw[u] = zq[row + h * dk + i];
      else if (i < 2 * dk) raw[u] = zf[row + h * dk + i - dk];
      else if (i < 2 * dk + ncol) raw[u] = v[row + h * dv + col0 + i - 2 * dk];
    }
  };
  auto commit = [&](float* dst) {
#pragma unroll
    for (int u = 0; u < kScanPF; ++u) {
      const int i = threadIdx.x + u * 256;
      if (i < in_len) {
        const float z = Cvt<T>::to_f32(raw[u]);
        float r = z;                                              // value column
        if (i < dk) r = z * sigmoidf_(z);                         // q = silu(zq)
        else if (i < 2 * dk) r = low_r[u] + (1.0f - low_r[u]) * sigmoidf_(z + bias_r[u]);
        dst[i] = r;
      }
    }
  };
  fetch(0);
  commit(in_s);
  __syncthreads();
  for (int t = 0; t < sq.count; ++t) {
    const float* cur = in_s + (t & 1) * in_len;
    if (t + 1 < sq.count) fetch(t + 1);
    {
      const float vc = cur[2 * dk + c];
      float sum = 0.f;
      for (int i = rg; i < dk; i += kScanRG) {
        const float f = cur[dk + i];
        const float s_new = f * S[i * kScanCols + c] + (1.0f - f) * vc;
        S[i * kScanCols + c] = s_new;
        sum = fmaf(s_new, cur[i], sum);
      }
      part[rg * kScanCols + c] = sum;
    }
    if (t + 1 < sq.count) commit(in_s + ((t + 1) & 1) * in_len);
    __syncthreads();
    if (rg == 0 && c < ncol) {
      float o = 0.f;
#pragma unroll
      for (int r = 0; r < kScanRG; ++r) o += part[r * kScanCols + c];
      o_raw[(static_cast<int64_t>(sq.tok0 + t) * H + h) * dv + col0 + c] = o;
    }
    __syncthreads();
  }
  for (int i = threadIdx.x; i < dk * kScanCols; i += blockDim.x) {
    const int r = i / kScanCols, cc = i - r * kScanCols;
    if (cc < ncol) st[r * dv + col0 + cc] = S[i];
  }
}

// Register form for key sizes up to 128: four adjacent lanes share a value column, lane r of the four keeps the state
// rows i = r, r + 4, ... of that column in REGISTERS for the whole portion.  A token costs dk / 4 state updates per
// thread, two shuffles to add the four partial read-outs, and no barrier; q and f of a token are broadcast reads
// from shared memory, stored there grouped by r.  The CTA (128 threads = 32 columns) stages the activated inputs of
// 4 tokens at a time, double buffered: raw loads of the next 4 tokens are issued before the current 4 are
// computed and converted afterwards, one barrier per 4 tokens.  The summation order of a read-out is fixed by dk.
constexpr int kScanChunk = 4;
constexpr int kScanNT = 128;
constexpr int kScanColsR = kScanNT / 4;   // value columns per CTA

template <typename T, int DK>
__global__ void __launch_bounds__(kScanNT)
gated_scan_columns_kernel(float* __restrict__ o_raw, const T* __restrict__ zq, const T* __restrict__ zf,
                          const T* __restrict__ v, int64_t in_stride, const T* __restrict__ f_bias,
                          const T* __restrict__ lower, float* __restrict__ state, const ScanSeq* __restrict__ seqs, int H,
                          int dk, int dv) {
  extern __shared__ __align__(16) float smem[];
  constexpr int RW4 = DK / 4;                           // state rows per thread
  const ScanSeq sq = seqs[blockIdx.x];
  const int h = blockIdx.y;
  const int r = threadIdx.x & 3;
  const int cl = threadIdx.x >> 2;                       // column within the CTA
  const int col0 = blockIdx.z * kScanColsR;
  const int col = col0 + cl;
  const bool has_col = col < dv;
  const int ncol = min(kScanColsR, dv - col0);
  constexpr int row_len = 2 * DK + kScanColsR;           // q grouped by r [4][RW4] | f likewise | v[32]
  float* buf0 = smem;
  float* buf1 = smem + kScanChunk * row_len;
  float* st = state + (static_cast<int64_t>(sq.slot) * H + h) * dk * dv;
  float S[RW4];
  // the CTA's slab of the state ([dk][32 columns]) moves through shared memory so that global rows are read and
  // written as whole 128-byte segments; the staging buffers are free at both ends of the kernel
  if (!sq.fresh) {
    for (int idx = threadIdx.x; idx < dk * kScanColsR; idx += kScanNT) {
      const int i = idx / kScanColsR, c = idx - i * kScanColsR;
      smem[idx] = c < ncol ? st[i * dv + col0 + c] : 0.f;
    }
    __syncthreads();
  }
#pragma unroll
  for (int k = 0; k < RW4; ++k) {
    const int i = 4 * k + r;
    S[k] = (!sq.fresh && i < dk) ? smem[i * kScanColsR + cl] : 0.f;
  }
  __syncthreads();
  constexpr int kPer = (kScanChunk * row_len + kScanNT - 1) / kScanNT;   // staged elements per thread and chunk
  T raw[kPer];
  // staged element e of a chunk: token e / row_len, slot s = e % row_len; slots [0, DK) hold q with slot = r * RW4 + k
  // for row i = 4 k + r, slots [DK, 2 DK) hold f the same way, the rest the CTA's value columns
  auto fetch = [&](int t0) {
#pragma unroll
    for (int u = 0; u < kPer; ++u) {
      const int e = threadIdx.x + u * kScanNT;
      const int tt = e / row_len, sl = e - tt * row_len;
      raw[u] = Cvt<T>::from_f32(0.f);
      if (tt < kScanChunk && t0 + tt < sq.count) {
        const int64_t row = static_cast<int64_t>(sq.tok0 + t0 + tt) * in_stride;
        if (sl < 2 * DK) {
          const int s2 = sl < DK ? sl : sl - DK;
          const int i = 4 * (s2 % RW4) + s2 / RW4;
          if (i < dk) raw[u] = sl < DK ? zq[row + h * dk + i] : zf[row + h * dk + i];
        } else if (sl - 2 * DK < ncol) {
          raw[u] = v[row + h * dv + col0 + sl - 2 * DK];
        }
      }
    }
  };
  auto commit = [&](float* dst, int n_valid) {   // tokens beyond the portion are not activated (nor read later)
#pragma unroll
    for (int u = 0; u < kPer; ++u) {
      const int e = threadIdx.x + u * kScanNT;
      const int tt = e / row_len, sl = e - tt * row_len;
      if (tt < n_valid) {
        const float z = Cvt<T>::to_f32(raw[u]);
        float val = z;
        if (sl < DK) {
          val = z * sigmoidf_(z);
        } else if (sl < 2 * DK) {
          const int s2 = sl - DK;
          const int i = 4 * (s2 % RW4) + s2 / RW4;
          val = 0.f;   // padded rows: f = 0 and q = 0, they never reach a read-out
          if (i < dk) {
            const float lo = Cvt<T>::to_f32(lower[h * dk + i]);
            val = lo + (1.0f - lo) * sigmoidf_(z + Cvt<T>::to_f32(f_bias[h * dk + i]));
          }
        }
        dst[e] = val;
      }
    }
  };
  fetch(0);
  commit(buf0, min(kScanChunk, sq.count));
  __syncthreads();
  for (int t0 = 0; t0 < sq.count; t0 += kScanChunk) {
    const float* cur = ((t0 / kScanChunk) & 1) ? buf1 : buf0;
    float* nxt = ((t0 / kScanChunk) & 1) ? buf0 : buf1;
    const bool more = t0 + kScanChunk < sq.count;
    if (more) fetch(t0 + kScanChunk);
    const int n_here = min(kScanChunk, sq.count - t0);
    for (int tt = 0; tt < n_here; ++tt) {
      const float* row = cur + tt * row_len;
      const float vc = row[2 * DK + cl];
      const float* qr = row + r * RW4;
      const float* fr = row + DK + r * RW4;
      float o0 = 0.f, o1 = 0.f;
#pragma unroll
      for (int k = 0; k < RW4; k += 4) {
        const float4 q4 = *reinterpret_cast<const float4*>(qr + k);
        const float4 f4 = *reinterpret_cast<const float4*>(fr + k);
        S[k] = f4.x * S[k] + (1.0f - f4.x) * vc;
        o0 = fmaf(S[k], q4.x, o0);
        S[k + 1] = f4.y * S[k + 1] + (1.0f - f4.y) * vc;
        o1 = fmaf(S[k + 1], q4.y, o1);
        S[k + 2] = f4.z * S[k + 2] + (1.0f - f4.z) * vc;
        o0 = fmaf(S[k + 2], q4.z, o0);
        S[k + 3] = f4.w * S[k + 3] + (1.0f - f4.w) * vc;
        o1 = fmaf(S[k + 3], q4.w, o1);
      }
      float o = o0 + o1;
      o += __shfl_xor_sync(0xffffffffu, o, 1);
      o += __shfl_xor_sync(0xffffffffu, o, 2);
      if (r == 0 && has_col) o_raw[(static_cast<int64_t>(sq.tok0 + t0 + tt) * H + h) * dv + col] = o;
    }
    if (more) commit(nxt, min(kScanChunk, sq.count - t0 - kScanChunk));
    __syncthreads();
  }
#pragma unroll
  for (int k = 0; k < RW4; ++k) {
    const int i = 4 * k + r;
    if (i < dk) smem[i * kScanColsR + cl] = S[k];
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < dk * kScanColsR; idx += kScanNT) {
    const int i = idx / kScanColsR, c = idx - i * kScanColsR;
    if (c < ncol) st[i * dv + col0 + c] = smem[idx];
  }
}

// per-head weighted RMS norm of fp32 rows [rows, dv] -> T; one warp per row
template <typename T>
__global__ void __launch_bounds__(256)
head_rmsnorm_kernel(T* __restrict__ out, const float* __restrict__ x, const T* __restrict__ w, float eps, int64_t rows,
                    int dv) {
  const int64_t row = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int lane = threadIdx.x & 31;
  const float* xr = x + row * dv;
  float ss = 0.f;
  for (int c = lane; c < dv; c += 32) ss = fmaf(xr[c], xr[c], ss);
  const float inv = rsqrtf(warp_sum(ss) / static_cast<float>(dv) + eps);
  for (int c = lane; c < dv; c += 32) out[row * dv + c] = Cvt<T>::from_f32(xr[c] * inv * Cvt<T>::to_f32(w[c]));
}

// ---- PolyNorm ---------------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256)
polynorm_kernel(T* __restrict__ out, const T* __restrict__ z, int64_t z_stride, const T* __restrict__ coef, float eps,
                int ff) {
  __shared__ float red[32];
  const T* zr = z + static_cast<int64_t>(blockIdx.x) * z_stride;
  float s1 = 0.f, s2 = 0.f, s3 = 0.f;
  for (int i = threadIdx.x; i < ff; i += blockDim.x) {
    const float a = Cvt<T>::to_f32(zr[i]);
    const float a2 = a * a, a3 = a2 * a;
    s1 = fmaf(a, a, s1);
    s2 = fmaf(a2, a2, s2);
    s3 = fmaf(a3, a3, s3);
  }
  const float n = static_cast<float>(ff);
  const float i1 = rsqrtf(block_sum_256(s1, red) / n + eps);
  const float i2 = rsqrtf(block_sum_256(s2, red) / n + eps);
  const float i3 = rsqrtf(block_sum_256(s3, red) / n + eps);
  const float ca = Cvt<T>::to_f32(coef[0]), cb = Cvt<T>::to_f32(coef[1]), cc = Cvt<T>::to_f32(coef[2]),
              ce = Cvt<T>::to_f32(coef[3]);
  T* orow = out + static_cast<int64_t>(blockIdx.x) * ff;
  for (int i = threadIdx.x; i < ff; i += blockDim.x) {
    const float a = Cvt<T>::to_f32(zr[i]);
    const float a2 = a * a;
    orow[i] = Cvt<T>::from_f32(ca * a * i1 + cb * a2 * i2 + cc * a2 * a * i3 + ce);
  }
}

// ---- routing ----------------------------------------------------------------------------------------------------
// One warp per token: the `top` largest logits (ties: lowest index), weight = sigmoid(logit).
__global__ void __launch_bounds__(128)
sigmoid_topk_kernel(int32_t* __restrict__ ids, float* __restrict__ weights, const float* __restrict__ logits, int n_tok,
                    int E, int top) {
  const int tok = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (tok >= n_tok) return;
  const int lane = threadIdx.x & 31;
  const float* z = logits + static_cast<int64_t>(tok) * E;
  for (int k = 0; k < top; ++k) {
    float best = -INFINITY;
    int bi = 0x7fffffff;
    for (int e = lane; e < E; e += 32) {
      bool taken = false;
      for (int j = 0; j < k; ++j) taken |= ids[static_cast<int64_t>(tok) * top + j] == e;
      const float f = z[e];
      if (!taken && (f > best || (f == best && e < bi))) {
        best = f;
        bi = e;
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ob > best || (ob == best && oi < bi)) {
        best = ob;
        bi = oi;
      }
    }
    if (lane == 0) {
      ids[static_cast<int64_t>(tok) * top + k] = bi;
      weights[static_cast<int64_t>(tok) * top + k] = sigmoidf_(best);
    }
    __syncwarp();
  }
}

// rows of the expert-sorted input: xs[r] = T(w[src[r]] * h[src[r] / top])
template <typename T>
__global__ void __launch_bounds__(256)
scaled_gather_kernel(T* __restrict__ xs, const T* __restrict__ h, const float* __restrict__ weights,
                     const int64_t* __restrict__ src, int top, int width) {
  const int64_t pair = src[blockIdx.x];
  const float w = weights[pair];
  const T* hr = h + (pair / top) * width;
  T* o = xs + static_cast<int64_t>(blockIdx.x) * width;
  for (int i = threadIdx.x; i < width; i += blockDim.x) o[i] = Cvt<T>::from_f32(w * Cvt<T>::to_f32(hr[i]));
}

// y = g' * sigmoid(alpha g') * (u' + 1), g' = min(g, limit), u' = clamp(u, -limit, limit); gu rows hold g | u
template <typename T>
__global__ void __launch_bounds__(256)
clamped_glu_kernel(T* __restrict__ y, const T* __restrict__ gu, int64_t rows, int ff, float limit, float alpha) {
  const int64_t n = rows * ff;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t r = i / ff;
    const int c = static_cast<int>(i - r * ff);
    const float g = fminf(Cvt<T>::to_f32(gu[r * 2 * ff + c]), limit);
    const float u = fminf(fmaxf(Cvt<T>::to_f32(gu[r * 2 * ff + ff + c]), -limit), limit);
    y[i] = Cvt<T>::from_f32(g * sigmoidf_(alpha * g) * (u + 1.0f));
  }
}

// out[n] = sum_k ys[where[n * top + k]] in fp32, k ascending
template <typename T>
__global__ void __launch_bounds__(256)
expert_combine_kernel(float* __restrict__ out, const T* __restrict__ ys, const int64_t* __restrict__ where, int top,
                      int width) {
  const int64_t n = blockIdx.x;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    float a = 0.f;
    for (int k = 0; k < top; ++k) a += Cvt<T>::to_f32(ys[where[n * top + k] * width + i]);
    out[n * width + i] = a;
  }
}

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" {

int b200_mixers_abi_version(void) { return B200_MIXERS_ABI_VERSION; }

const char* b200_mixers_last_error(void) { return last_error_buf(); }

int b200_offset_rmsnorm(void* out, const float* x, const void* weight, float eps, int rows, int width, int dtype,
                        void* stream) {
  if (rows < 0 || width <= 0) return fail(B200_EINVAL, "b200_offset_rmsnorm: bad sizes");
  if (rows == 0) return 0;
  if (!out || !x || !weight) return fail(B200_EINVAL, "b200_offset_rmsnorm: null pointer");
  return mixer_by_dtype(dtype, "b200_offset_rmsnorm", [&](auto* tag) {
    using T = std::remove_pointer_t<decltype(tag)>;
    offset_rmsnorm_kernel<T><<<rows, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<T*>(out), x, static_cast<const T*>(weight), eps, width);
    return check_launch("b200_offset_rmsnorm");
  });
}

int b200_postnorm_residual(float* x, const void* y, int64_t y_stride, int y_is_f32, const void* w_post, float mult,
                           const void* w_next, void* out_next, float eps, int rows, int width, int dtype, void* stream) {
  if (rows < 0 || width <= 0 || width > 40000) return fail(B200_EINVAL, "b200_postnorm_residual: bad sizes");
  if (rows == 0) return 0;
  if (!x || !y || !w_post || (w_next && !out_next)) return fail(B200_EINVAL, "b200_postnorm_residual: null pointer");
  const size_t smem = static_cast<size_t>(width) * sizeof(float);
  return mixer_by_dtype(dtype, "b200_postnorm_residual", [&](auto* tag) {
    using T = std::remove_pointer_t<decltype(tag)>;
    auto launch = [&](auto kern, auto* ytag) {
      using Y = std::remove_pointer_t<decltype(ytag)>;
      if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
      kern<<<rows, 256, smem, static_cast<cudaStream_t>(stream)>>>(x, static_cast<const Y*>(y), y_stride,
                                                                  static_cast<const T*>(w_post), mult,
                                                                  static_cast<const T*>(w_next), static_cast<T*>(out_next),
                                                                  eps, width);
    };
    if (y_is_f32) launch(postnorm_residual_kernel<T, float>, static_cast<float*>(nullptr));
    else launch(postnorm_residual_kernel<T, T>, static_cast<T*>(nullptr));
    return check_launch("b200_postnorm_residual");
  });
}

int b200_value_prep_append(const void* k, int64_t k_stride, const void* v, int64_t v_stride, const void* v_prev,
                           void* v_keep, float lam, float eps, void* k_pool, void* v_pool, const int64_t* slot_mapping,
                           int n_tok, int G, int dk, int dv, int block_size, int64_t max_blocks, int dtype, void* stream) {
  if (n_tok < 0 || G <= 0 || dk <= 0 || dv <= 0 || block_size <= 0) return fail(B200_EINVAL, "b200_value_prep_append: bad sizes");
  if (n_tok == 0) return 0;
  if (!k || !v || !k_pool || !v_pool || !slot_mapping) return fail(B200_EINVAL, "b200_value_prep_append: null pointer");
  return mixer_by_dtype(dtype, "b200_value_prep_append", [&](auto* tag) {
    using T = std::remove_pointer_t<decltype(tag)>;
    value_prep_append_kernel<T><<<n_tok, 128, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const T*>(k), k_stride, static_cast<const T*>(v), v_stride, static_cast<const T*>(v_prev),
        static_cast<T*>(v_keep), lam, eps, static_cast<T*>(k_pool), static_cast<T*>(v_pool), slot_mapping, G, dk, dv,
        block_size, max_blocks);
    return check_launch("b200_value_prep_append");
  });
}

int b200_biased_attn_tile_tokens(int n_tokens_in_portion, int H, int G) {
  // tokens per CTA: prompt portions fill 8 warps x 4 rows, a decoded token takes what its head group needs
  const int rep = std::max(1, H / std::max(G, 1));
  const int rows_max = kAttnWarps * 4;
  return std::max(1, std::min(n_tokens_in_portion, rows_max / std::min(rep, rows_max)));
}

int b200_biased_paged_attn(void* out, const void* q, int64_t q_stride, const void* gate, int64_t gate_stride,
                           const void* k_pool, const void* v_pool, const int32_t* block_tables, int table_stride,
                           const int32_t* tiles, int n_tiles, int max_tile_tokens, const int32_t* tok_pos,
                           const float* bias_lut, int lut_len, float scale, float temp_coef, int temp_every, int H, int G,
                           int dk, int dv, int block_size, int dtype, void* stream) {
  if (n_tiles < 0 || H <= 0 || G <= 0 || H % G || dk <= 0 || dv <= 0 || dv > 256 || block_size <= 0 || lut_len <= 0 ||
      max_tile_tokens <= 0)
    return fail(B200_EINVAL, "b200_biased_paged_attn: bad sizes");
  if (n_tiles == 0) return 0;
  if (!out || !q || !k_pool || !v_pool || !block_tables || !tiles || !tok_pos || !bias_lut)
    return fail(B200_EINVAL, "b200_biased_paged_attn: null pointer");
  const int rep = H / G;
  const int rows = max_tile_tokens * rep;
  if (rows > kAttnWarps * 4) return fail(B200_ESHAPE, "b200_biased_paged_attn: %d rows per tile > %d", rows, kAttnWarps * 4);
  const int dkp = (dk + 3) & ~3;
  const int rw = rows <= kAttnWarps ? 1 : (rows <= 2 * kAttnWarps ? 2 : 4);  // rows per warp (template RW)
  const size_t smem = sizeof(float) * (static_cast<size_t>(kKeyTile) * (dkp + 4) + static_cast<size_t>(kKeyTile) * dv +
                                       static_cast<size_t>(kAttnWarps) * rw * dkp);
  if (smem > 200 * 1024) return fail(B200_ESHAPE, "b200_biased_paged_attn: head sizes %d / %d need too much shared memory", dk, dv);
  const dim3 grid(n_tiles, G);
  return mixer_by_dtype(dtype, "b200_biased_paged_attn", [&](auto* tag) {
    using T = std::remove_pointer_t<decltype(tag)>;
    auto launch = [&](auto kern) {
      if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
      kern<<<grid, kAttnWarps * 32, smem, static_cast<cudaStream_t>(stream)>>>(
          static_cast<T*>(out), static_cast<const T*>(q), q_stride, static_cast<const T*>(gate), gate_stride,
          static_cast<const T*>(k_pool), static_cast<const T*>(v_pool), block_tables, table_stride,
          reinterpret_cast<const AttnTile*>(tiles), tok_pos, bias_lut, lut_len, scale, temp_coef, temp_every, H, G, dk, dv,
          block_size);
    };
    const int dvl = (dv + 31) / 32;
    // 16-byte chunk loads with a one-tile register prefetch when rows are multiples of 16 bytes and a tile's chunks
    // fit 4 (or 8) per thread; element-wise loads otherwise
    constexpr int VN = 16 / static_cast<int>(sizeof(T));
    const bool vec = dk % VN == 0 && dv % VN == 0 && aligned16(k_pool) && aligned16(v_pool);
    const int per_thread = vec ? (kKeyTile * (dk / VN + dv / VN) + kAttnWarps * 32 - 1) / (kAttnWarps * 32) : 0;
    const int nch = !vec || per_thread > 8 ? 0 : (per_thread <= 4 ? 4 : 8);
#define B200_ATTN_DV(RW_, NCH_)                                              \
  if (dvl <= 1) launch(biased_paged_attn_kernel<T, RW_, 1, NCH_>);           \
  else if (dvl <= 2) launch(biased_paged_attn_kernel<T, RW_, 2, NCH_>);      \
  else if (dvl <= 4) launch(biased_paged_attn_kernel<T, RW_, 4, NCH_>);      \
  else launch(biased_paged_attn_kernel<T, RW_, 8, NCH_>);
#define B200_ATTN_CASE(RW_)                                                  \
  if (nch == 4) { B200_ATTN_DV(RW_, 4) }                                     \
  else if (nch == 8) { B200_ATTN_DV(RW_, 8) }                                \
  else { B200_ATTN_DV(RW_, 0) }
    if (rw <= 1) { B200_ATTN_CASE(1) }
    else if (rw <= 2) { B200_ATTN_CASE(2) }
    else { B200_ATTN_CASE(4) }
#undef B200_ATTN_CASE
#undef B200_ATTN_DV
    return check_launch("b200_biased_paged_attn");
  });
}

int b200_biased_prompt_attn_tile_tokens(int H, int G) { return std::max(1, kMmaRows / std::max(1, H / std::max(G, 1))); }

int b200_biased_prompt_attn_supported(int dk, int dv, int dtype) {
  return (dtype == B200_DTYPE_BF16 || dtype == B200_DTYPE_F16) && dk > 0 && dk % 16 == 0 && dk <= 256 && dv > 0 &&
         dv % 8 == 0 && dv <= 128;
}

int b200_biased_prompt_attn(void* out, const void* q, int64_t q_stride, const void* gate, int64_t gate_stride,
                            const void* k_pool, const void* v_pool, const int32_t* block_tables, int table_stride,
                            const int32_t* tiles, int n_tiles, int max_tile_tokens, const int32_t* tok_pos, const float* bias_lut,
                            int lut_len, float scale, float temp_coef, int temp_every, int H, int G, int dk, int dv,
                            int block_size, int dtype, void* stream) {
  if (n_tiles < 0 || H <= 0 || G <= 0 || H % G || block_size <= 0 || lut_len <= 0)
    return fail(B200_EINVAL, "b200_biased_prompt_attn: bad sizes");
  if (!b200_biased_prompt_attn_supported(dk, dv, dtype))
    return fail(B200_ESHAPE, "b200_biased_prompt_attn: needs a 16-bit dtype, dk %% 16 == 0 (<= 256), dv %% 8 == 0 (<= 128)");
  if (n_tiles == 0) return 0;
  if (!out || !q || !k_pool || !v_pool || !block_tables || !tiles || !tok_pos || !bias_lut)
    return fail(B200_EINVAL, "b200_biased_prompt_attn: null pointer");
  if (!aligned16(k_pool) || !aligned16(v_pool))
    return fail(B200_ESHAPE, "b200_biased_prompt_attn: pools must be 16-byte aligned");
  const int q_vec = aligned16(q) && (q_stride * 2) % 16 == 0;
  const int dv8 = dv <= 32 ? 4 : (dv <= 64 ? 8 : 16);
  const size_t tiles_bytes = 2u * (static_cast<size_t>(kMmaRows) * (dk + 8) * 3 + 2u * kMmaKeys * (dv8 * 8 + 8));
  const int rep = H / G;
  if (rep > kMmaRows) return fail(B200_ESHAPE, "b200_biased_prompt_attn: %d heads per kv head > %d", rep, kMmaRows);
  // the group's bias tables go to shared memory when they are small enough to leave room for two CTAs per SM
  const size_t lut_bytes = static_cast<size_t>(rep) * lut_len * 4;
  const int lut_in_smem = lut_bytes <= 20 * 1024;
  const size_t smem = tiles_bytes + (lut_in_smem ? lut_bytes : 0);
  const dim3 grid(n_tiles, G);
  return mixer_by_dtype(dtype, "b200_biased_prompt_attn", [&](auto* tag) {
    using T = std::remove_pointer_t<decltype(tag)>;
    if constexpr (std::is_same_v<T, float>) {
      return fail(B200_ESHAPE, "b200_biased_prompt_attn: 16-bit dtypes only");
    } else {
      auto launch = [&](auto kern) {
        if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
        kern<<<grid, 128, smem, static_cast<cudaStream_t>(stream)>>>(
            static_cast<T*>(out), static_cast<const T*>(q), q_stride, static_cast<const T*>(gate), gate_stride,
            static_cast<const T*>(k_pool), static_cast<const T*>(v_pool), block_tables, table_stride,
            reinterpret_cast<const AttnTile*>(tiles), tok_pos, bias_lut, lut_len, lut_in_smem, q_vec, scale, temp_coef,
            temp_every, H, G, dk, dv, block_size);
      };
      // tiles of at most 16 rows (decoded tokens): the four warps split the keys instead of the rows
      const bool ksplit = max_tile_tokens > 0 && max_tile_tokens * rep <= 16;
      if (ksplit) {
        if (dv8 == 4) launch(biased_prompt_attn_mma_kernel<T, 4, true>);
        else if (dv8 == 8) launch(biased_prompt_attn_mma_kernel<T, 8, true>);
        else launch(biased_prompt_attn_mma_kernel<T, 16, true>);
      } else {
        if (dv8 == 4) launch(biased_prompt_attn_mma_kernel<T, 4, false>);
        else if (dv8 == 8) launch(biased_prompt_attn_mma_kernel<T, 8, false>);
        else launch(biased_prompt_attn_mma_kernel<T, 16, false>);
      }
      return check_launch("b200_biased_prompt_attn");
    }
  });
}

int b200_grouped_linear_supported(int K, int dtype) {
  return (dtype == B200_DTYPE_BF16 || dtype == B200_DTYPE_F16) && K > 0 && K % 8 == 0;
}

int b200_grouped_linear(void* out, const void* xs, const void* w, const int32_t* offsets, int64_t max_rows, int E, int N,
                        int K, int dtype, void* stream) {
  if (max_rows < 0 || E <= 0 || N <= 0 || K <= 0) return fail(B200_EINVAL, "b200_grouped_linear: bad sizes");
  if (!b200_grouped_linear_supported(K, dtype))
    return fail(B200_ESHAPE, "b200_grouped_linear: needs a 16-bit dtype and K %% 8 == 0");
  if (max_rows == 0) return 0;
  if (!out || !xs || !w || !offsets) return fail(B200_EINVAL, "b200_grouped_linear: null pointer");
  if (!aligned16(xs) || !aligned16(w)) return fail(B200_ESHAPE, "b200_grouped_linear: operands must be 16-byte aligned");
  const int64_t zt = (max_rows + kGrpRows - 1) / kGrpRows;
  if (zt > 65535 || E > 65535) return fail(B200_ENOSPC, "b200_grouped_linear: %lld row tiles / %d experts beyond the grid", static_cast<long long>(zt), E);
  const size_t smem = 2u * 2u * (kGrpRows + kGrpCols) * (kGrpK + 8);
  const dim3 grid((N + kGrpCols - 1) / kGrpCols, E, static_cast<unsigned>(zt));
  return mixer_by_dtype(dtype, "b200_grouped_linear", [&](auto* tag) {
    using T = std::remove_pointer_t<decltype(tag)>;
    if constexpr (std::is_same_v<T, float>) {
      return fail(B200_ESHAPE, "b200_grouped_linear: 16-bit dtypes only");
    } else {
      auto kern = grouped_linear_kernel<T>;
      cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
      kern<<<grid, 128, smem, static_cast<cudaStream_t>(stream)>>>(static_cast<T*>(out), static_cast<const T*>(xs),
                                                                  static_cast<const T*>(w), offsets, N, K);
      return check_launch("b200_grouped_linear");
    }
  });
}

int b200_gated_scan(float* o_raw, const void* zq, const void* zf, const void* v, int64_t in_stride, const void* f_bias,
                    const void* lower, float* state, const int32_t* seqs, int n_seqs, int max_count, int H, int dk, int dv,
                    int dtype, void* stream) {
  if (n_seqs < 0 || H <= 0 || dk <= 0 || dv <= 0) return fail(B200_EINVAL, "b200_gated_scan: bad sizes");
  if (n_seqs == 0) return 0;
  if (!o_raw || !zq || !zf || !v || !f_bias || !lower || !state || !seqs) return fail(B200_EINVAL, "b200_gated_scan: null pointer");
  if (dk <= 128 && max_count >= 8) {
    // register kernel: 32 value columns per CTA, four lanes per column
    const int dkt = dk <= 16 ? 16 : (dk <= 32 ? 32 : (dk <= 64 ? 64 : 128));
    // the staging buffers double as the [dk][32] slab the state moves through at both ends of the kernel
    const size_t smem_c = sizeof(float) * std::max<size_t>(2 * kScanChunk * (2 * static_cast<size_t>(dkt) + kScanColsR),
                                                           static_cast<size_t>(dkt) * kScanColsR);
    const dim3 grid_c(n_seqs, H, (dv + kScanColsR - 1) / kScanColsR);
    return mixer_by_dtype(dtype, "b200_gated_scan", [&](auto* tag) {
      using T = std::remove_pointer_t<decltype(tag)>;
      auto launch = [&](auto kern) {
        kern<<<grid_c, kScanNT, smem_c, static_cast<cudaStream_t>(stream)>>>(
            o_raw, static_cast<const T*>(zq), static_cast<const T*>(zf), static_cast<const T*>(v), in_stride,
            static_cast<const T*>(f_bias), static_cast<const T*>(lower), state, reinterpret_cast<const ScanSeq*>(seqs), H,
            dk, dv);
      };
      if (dkt == 16) launch(gated_scan_columns_kernel<T, 16>);
      else if (dkt == 32) launch(gated_scan_columns_kernel<T, 32>);
      else if (dkt == 64) launch(gated_scan_columns_kernel<T, 64>);
      else launch(gated_scan_columns_kernel<T, 128>);
      return check_launch("b200_gated_scan");
    });
  }
  if (2 * dk + kScanCols > kScanPF * 256) return fail(B200_ESHAPE, "b200_gated_scan: key size %d beyond %d", dk, (kScanPF * 256 - kScanCols) / 2);
  const size_t smem = sizeof(float) * (static_cast<size_t>(dk) * kScanCols + 2 * (2 * static_cast<size_t>(dk) + kScanCols) +
                                       static_cast<size_t>(kScanRG) * kScanCols);
  const dim3 grid(n_seqs, H, (dv + kScanCols - 1) / kScanCols);
  return mixer_by_dtype(dtype, "b200_gated_scan", [&](auto* tag) {
    using T = std::remove_pointer_t<decltype(tag)>;
    auto kern = gated_scan_kernel<T>;
    if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    kern<<<grid, 256, smem, static_cast<cudaStream_t>(stream)>>>(
        o_raw, static_cast<const T*>(zq), static_cast<const T*>(zf), static_cast<const T*>(v), in_stride,
        static_cast<const T*>(f_bias), static_cast<const T*>(lower), state, reinterpret_cast<const ScanSeq*>(seqs), H, dk,
        dv);
    return check_launch("b200_gated_scan");
  });
}

int b200_head_rmsnorm(void* out, const float* x, const void* weight, float eps, int64_t rows, int dv, int dtype,
                      void* stream) {
  if (rows < 0 || dv <= 0) return fail(B200_EINVAL, "b200_head_rmsnorm: bad sizes");
  if (rows == 0) return 0;
  if (!out || !x || !weight) return fail(B200_EINVAL, "b200_head_rmsnorm: null pointer");
  return mixer_by_dtype(dtype, "b200_head_rmsnorm", [&](auto* tag) {
    using T = std::remove_pointer_t<decltype(tag)>;
    head_rmsnorm_kernel<T><<<static_cast<unsigned>((rows + 7) / 8), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<T*>(out), x, static_cast<const T*>(weight), eps, rows, dv);
    return check_launch("b200_head_rmsnorm");
  });
}

int b200_polynorm(void* out, const void* z, int64_t z_stride, const void* coef, float eps, int rows, int ff, int dtype,
                  void* stream) {
  if (rows < 0 || ff <= 0) return fail(B200_EINVAL, "b200_polynorm: bad sizes");
  if (rows == 0) return 0;
  if (!out || !z || !coef) return fail(B200_EINVAL, "b200_polynorm: null pointer");
  return mixer_by_dtype(dtype, "b200_polynorm", [&](auto* tag) {
    using T = std::remove_pointer_t<decltype(tag)>;
    polynorm_kernel<T><<<rows, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<T*>(out), static_cast<const T*>(z), z_stride, static_cast<const T*>(coef), eps, ff);
    return check_launch("b200_polynorm");
  });
}

int b200_sigmoid_topk(int32_t* ids, float* weights, const float* logits, int n_tok, int E, int top, void* stream) {
  if (n_tok < 0 || E <= 0 || top <= 0 || top > E) return fail(B200_EINVAL, "b200_sigmoid_topk: bad sizes");
  if (n_tok == 0) return 0;
  if (!ids || !weights || !logits) return fail(B200_EINVAL, "b200_sigmoid_topk: null pointer");
  sigmoid_topk_kernel<<<(n_tok + 3) / 4, 128, 0, static_cast<cudaStream_t>(stream)>>>(ids, weights, logits, n_tok, E, top);
  return check_launch("b200_sigmoid_topk");
}

int b200_scaled_gather(void* xs, const void* h, const float* weights, const int64_t* src, int64_t n_rows, int top,
                       int width, int dtype, void* stream) {
  if (n_rows < 0 || top <= 0 || width <= 0) return fail(B200_EINVAL, "b200_scaled_gather: bad sizes");
  if (n_rows == 0) return 0;
  if (!xs || !h || !weights || !src) return fail(B200_EINVAL, "b200_scaled_gather: null pointer");
  return mixer_by_dtype(dtype, "b200_scaled_gather", [&](auto* tag) {
    using T = std::remove_pointer_t<decltype(tag)>;
    scaled_gather_kernel<T><<<static_cast<unsigned>(n_rows), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<T*>(xs), static_cast<const T*>(h), weights, src, top, width);
    return check_launch("b200_scaled_gather");
  });
}

int b200_clamped_glu(void* y, const void* gu, int64_t rows, int ff, float limit, float alpha, int dtype, void* stream) {
  if (rows < 0 || ff <= 0) return fail(B200_EINVAL, "b200_clamped_glu: bad sizes");
  if (rows == 0) return 0;
  if (!y || !gu) return fail(B200_EINVAL, "b200_clamped_glu: null pointer");
  const int64_t n = rows * ff;
  const unsigned grid = static_cast<unsigned>(std::min<int64_t>((n + 255) / 256, 148 * 16));
  return mixer_by_dtype(dtype, "b200_clamped_glu", [&](auto* tag) {
    using T = std::remove_pointer_t<decltype(tag)>;
    clamped_glu_kernel<T><<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<T*>(y), static_cast<const T*>(gu),
                                                                               rows, ff, limit, alpha);
    return check_launch("b200_clamped_glu");
  });
}

int b200_expert_combine(float* out, const void* ys, const int64_t* where, int64_t n_tok, int top, int width, int dtype,
                        void* stream) {
  if (n_tok < 0 || top <= 0 || width <= 0) return fail(B200_EINVAL, "b200_expert_combine: bad sizes");
  if (n_tok == 0) return 0;
  if (!out || !ys || !where) return fail(B200_EINVAL, "b200_expert_combine: null pointer");
  return mixer_by_dtype(dtype, "b200_expert_combine", [&](auto* tag) {
    using T = std::remove_pointer_t<decltype(tag)>;
    expert_combine_kernel<T><<<static_cast<unsigned>(n_tok), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        out, static_cast<const T*>(ys), where, top, width);
    return check_launch("b200_expert_combine");
  });
}

}  // extern "C"
