// Decode attention over cached rows that hold their values inside their keys (one row [c | r] per token and kv
// head: the key is the whole row of `dk` elements, the value its first `dv`), for rows wider than the split
// kernel of attention_decode.cu takes.  bfloat16, tensor cores (mma.sync m16n8k16): the query heads of a kv head
// are the 16 rows of a tile, so a row of the cache is read once for all of them.
//
// Grid (split, kv head x head tile, sequence); a block of eight warps walks its run of the visible keys 64 at a
// time: the tile's rows go to shared memory (zeros beyond the run), warp w takes the scores of keys 8 w .. 8 w + 7
// (two chains of products side by side, one over the even and one over the odd stretches of 32 elements),
// the tile's maxima and sums meet in shared memory, the probabilities (bfloat16) too, and warp w then adds
// P V into the value columns it owns (every eighth group of 16).  A block leaves its unnormalised outputs, maxima
// and sums (natural exponents) where attn_decode_plain_merge_kernel of attention_plain.cu joins the runs
// (and adds the sink and the gate).
#include "common.cuh"

namespace {

constexpr int LA_KEYS = 64;        // keys of a tile
constexpr int LA_WARPS = 8;
constexpr int LA_MAX_DK = 640;
constexpr int LA_CHUNKS = 5;       // groups of 16 value columns a warp owns at most (dv <= 640)

__device__ __forceinline__ uint32_t la_smem(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void la_ldm4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void la_ldm4t(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
// 16 bytes from global to shared memory without a register in between; `on` false: zeros
__device__ __forceinline__ void la_cp16(uint32_t dst, const void* src, bool on) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(on ? 16 : 0) : "memory");
}
__device__ __forceinline__ void la_mma(float* c, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
               "{%0, %1, %2, %3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__global__ void __launch_bounds__(LA_WARPS * 32)
attn_decode_latent_kernel(const __nv_bfloat16* __restrict__ q, long long q_stride, const __nv_bfloat16* __restrict__ kcache,
                          const int* __restrict__ page_table, int max_pages, const int* __restrict__ slots,
                          const int* __restrict__ lens, int nq, int nkv, int dk, int dv, float scale, int window,
                          int mask_kind, int ring_rows, int n_splits, float* __restrict__ part_o,
                          float* __restrict__ part_ml) {
  pdl_launch_dependents();
  extern __shared__ __align__(16) unsigned char la_raw[];
  const int pitch = dk + 8;                                     // elements of a row in shared memory (16-byte pieces shifted by 4 banks a row)
  __nv_bfloat16* q_s = reinterpret_cast<__nv_bfloat16*>(la_raw);            // [16][pitch]
  __nv_bfloat16* k_s = q_s + 16 * pitch;                                    // [64][pitch]
  __nv_bfloat16* p_s = k_s + LA_KEYS * pitch;                               // [16][72]
  float* max_s = reinterpret_cast<float*>(p_s + 16 * 72);                   // [warps][16]
  float* sum_s = max_s + LA_WARPS * 16;                                     // [warps][16]
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  const int split = blockIdx.x, b = blockIdx.z;
  const int group = nq / nkv, tiles = (group + 15) / 16;
  const int kvh = blockIdx.y / tiles, head0 = kvh * group + (blockIdx.y % tiles) * 16;
  const int n_heads = min(16, kvh * group + group - head0);
  const int slot = slots[b];
  const int pos = lens[b] - 1;
  // this block's run of the visible keys
  int lo = 0, hi = -1;
  if (slot >= 0 && pos >= 0) {
    lo = window <= 0 ? 0 : (mask_kind == AF_MASK_CHUNK ? pos - pos % window : max(0, pos - window + 1));
    const int per = (pos - lo + n_splits) / n_splits;
    lo += split * per;
    hi = min(pos, lo + per - 1);
  }
  pdl_wait();
  // ---- the queries of the tile's heads (rows of heads that are not there: zeros)
  const int pieces = dk / 8;
  for (int i = tid; i < 16 * pieces; i += blockDim.x) {
    const int r = i / pieces, c = i - r * pieces;
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (r < n_heads && hi >= lo) v = *reinterpret_cast<const uint4*>(q + (size_t)b * q_stride + (size_t)(head0 + r) * dk + c * 8);
    *reinterpret_cast<uint4*>(q_s + r * pitch + c * 8) = v;
  }
  const int n16 = dv / 16;                                      // groups of 16 value columns; warp w owns w, w + 8, ...
  float o[LA_CHUNKS][2][4];
#pragma unroll
  for (int c = 0; c < LA_CHUNKS; ++c)
#pragma unroll
    for (int n = 0; n < 2; ++n)
#pragma unroll
      for (int e = 0; e < 4; ++e) o[c][n][e] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};   // rows g and g + 8
  const int* pt = page_table + (size_t)max(slot, 0) * max_pages;
  for (int j0 = lo; j0 <= hi; j0 += LA_KEYS) {
    __syncthreads();                                            // the tile before is done with (and q_s is written)
    // ---- 64 rows of the cache, zeros beyond the run: a warp takes every eighth row, all copies in flight at once
    for (int r = warp; r < LA_KEYS; r += LA_WARPS) {
      const int j = j0 + r;
      const __nv_bfloat16* src = kcache;
      bool on = j <= hi;
      if (on) {
        const int rr = ring_rows > 0 ? j % ring_rows : j;
        on = AF_INDEX_OK(rr / AF_PAGE < max_pages && pt[rr / AF_PAGE] >= 0, rr);
        if (on) src = kcache + (((size_t)pt[rr / AF_PAGE] * nkv + kvh) * AF_PAGE + rr % AF_PAGE) * dk;
      }
      for (int c = lane; c < pieces; c += 32) la_cp16(la_smem(k_s + r * pitch + c * 8), src + (on ? c * 8 : 0), on);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();
    // ---- scores of this warp's 8 keys: one load brings a key tile's operands of 32 elements, two products
    float sa[4] = {0.f, 0.f, 0.f, 0.f}, sb[4] = {0.f, 0.f, 0.f, 0.f};
    for (int kk = 0; kk < dk; kk += 32) {
      uint32_t a0, a1, a2, a3, b0, b1, b2, b3;
      la_ldm4(la_smem(k_s + (warp * 8 + (lane & 7)) * pitch + kk + (lane >> 3) * 8), b0, b1, b2, b3);
      la_ldm4(la_smem(q_s + (lane & 15) * pitch + kk + (lane >> 4) * 8), a0, a1, a2, a3);
      la_mma(sa, a0, a1, a2, a3, b0, b1);
      if (kk + 16 < dk) {                                       // (dk is a multiple of 16: the last stretch may be half)
        la_ldm4(la_smem(q_s + (lane & 15) * pitch + kk + 16 + (lane >> 4) * 8), a0, a1, a2, a3);
        la_mma(sb, a0, a1, a2, a3, b2, b3);
      }
    }
    float s[4];
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int j = j0 + warp * 8 + 2 * t + (e & 1);
      s[e] = j <= hi ? (sa[e] + sb[e]) * scale : -INFINITY;
      mx[e >> 1] = fmaxf(mx[e >> 1], s[e]);
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
      if (t == 0) max_s[warp * 16 + g + 8 * r] = mx[r];
    }
    __syncthreads();
    float corr[2], ref[2], sm[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      const int row = g + 8 * r;
      float tile_max = max_s[row];
#pragma unroll
      for (int w2 = 1; w2 < LA_WARPS; ++w2) tile_max = fmaxf(tile_max, max_s[w2 * 16 + row]);
      const float m_new = fmaxf(m_run[r], tile_max);
      ref[r] = m_new == -INFINITY ? 0.f : m_new;
      corr[r] = m_run[r] == -INFINITY ? 0.f : __expf(m_run[r] - ref[r]);
      m_run[r] = m_new;
    }
    {
      const float p0 = __expf(s[0] - ref[0]), p1 = __expf(s[1] - ref[0]);
      const float p2 = __expf(s[2] - ref[1]), p3 = __expf(s[3] - ref[1]);
      const __nv_bfloat162 lo2 = __floats2bfloat162_rn(p0, p1), hi2 = __floats2bfloat162_rn(p2, p3);
      // (the sums take the rounded values that the product will see)
      sm[0] = __low2float(lo2) + __high2float(lo2);
      sm[1] = __low2float(hi2) + __high2float(hi2);
      *reinterpret_cast<__nv_bfloat162*>(p_s + g * 72 + warp * 8 + 2 * t) = lo2;
      *reinterpret_cast<__nv_bfloat162*>(p_s + (g + 8) * 72 + warp * 8 + 2 * t) = hi2;
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      sm[r] += __shfl_xor_sync(0xffffffffu, sm[r], 1);
      sm[r] += __shfl_xor_sync(0xffffffffu, sm[r], 2);
      if (t == 0) sum_s[warp * 16 + g + 8 * r] = sm[r];
    }
    __syncthreads();
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      const int row = g + 8 * r;
      float tile_sum = 0.f;
#pragma unroll
      for (int w2 = 0; w2 < LA_WARPS; ++w2) tile_sum += sum_s[w2 * 16 + row];
      l_run[r] = l_run[r] * corr[r] + tile_sum;
    }
    // ---- O += P V over the value columns this warp owns
#pragma unroll
    for (int c = 0; c < LA_CHUNKS; ++c) {
      const int chunk = warp + LA_WARPS * c;
      if (chunk < n16) {
#pragma unroll
        for (int n = 0; n < 2; ++n) {
          o[c][n][0] *= corr[0], o[c][n][1] *= corr[0];
          o[c][n][2] *= corr[1], o[c][n][3] *= corr[1];
        }
#pragma unroll
        for (int ks = 0; ks < LA_KEYS / 16; ++ks) {
          uint32_t a0, a1, a2, a3, b0, b1, b2, b3;
          la_ldm4(la_smem(p_s + (lane & 15) * 72 + ks * 16 + (lane >> 4) * 8), a0, a1, a2, a3);
          la_ldm4t(la_smem(k_s + (ks * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * pitch + chunk * 16 + (lane >> 4) * 8), b0, b1, b2, b3);
          la_mma(o[c][0], a0, a1, a2, a3, b0, b1);
          la_mma(o[c][1], a0, a1, a2, a3, b2, b3);
        }
      }
    }
  }
  // ---- this run's part of every head of the tile
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int row = g + 8 * r;
    if (row >= n_heads) continue;
    const size_t u = ((size_t)b * nq + head0 + row) * n_splits + split;
    if (warp == 0 && t == 0) part_ml[2 * u] = m_run[r], part_ml[2 * u + 1] = l_run[r];
#pragma unroll
    for (int c = 0; c < LA_CHUNKS; ++c) {
      const int chunk = warp + LA_WARPS * c;
      if (chunk < n16) {
#pragma unroll
        for (int n = 0; n < 2; ++n)
          *reinterpret_cast<float2*>(part_o + u * dv + chunk * 16 + n * 8 + 2 * t) = make_float2(o[c][n][2 * r], o[c][n][2 * r + 1]);
      }
    }
  }
}

}  // namespace

// 1 when the kernel takes these sizes.
AF_EXPORT int af_attn_decode_latent_supported(int dk, int dv) {
  return dk % 16 == 0 && dv % 16 == 0 && dv <= dk && dk <= LA_MAX_DK && dv / 16 <= LA_WARPS * LA_CHUNKS ? 1 : 0;
}

// The split pass alone: part_o [batch, nq, n_splits, dv] and part_ml [batch, nq, n_splits, 2] (maximum and sum,
// natural exponents; -inf and 0 for an empty run or a padding row) for af_attn_decode_plain's merge kernel.
AF_EXPORT int af_attn_decode_latent(const void* q, long long q_stride, const void* kcache, const int* page_table,
                                    int max_pages, const int* slots, const int* lens, int batch, int nq, int nkv, int dk,
                                    int dv, float scale, int window, int mask_kind, int ring_rows, int n_splits,
                                    float* part_o, float* part_ml, cudaStream_t stream) {
  if (batch == 0) return 0;
  AF_REQUIRE(nq > 0 && nkv > 0 && nq % nkv == 0 && batch < 65536, "af_attn_decode_latent: heads %d, groups %d", nq, nkv);
  AF_REQUIRE(af_attn_decode_latent_supported(dk, dv), "af_attn_decode_latent: rows of %d with values of %d", dk, dv);
  AF_REQUIRE(mask_kind == AF_MASK_WINDOW || mask_kind == AF_MASK_CHUNK, "af_attn_decode_latent: mask kind %d", mask_kind);
  AF_REQUIRE(ring_rows % AF_PAGE == 0 && (ring_rows == 0 || (window > 0 && window <= ring_rows)),
             "af_attn_decode_latent: window %d, ring rows %d", window, ring_rows);
  AF_REQUIRE(n_splits >= 1 && n_splits < 65536 && part_o != nullptr && part_ml != nullptr, "af_attn_decode_latent: splits %d", n_splits);
  AF_REQUIRE((((uintptr_t)q | (uintptr_t)kcache) & 15) == 0 && q_stride % 8 == 0, "af_attn_decode_latent: 16-byte aligned rows");
  const int tiles = (nq / nkv + 15) / 16;
  const size_t smem = (size_t)(16 + LA_KEYS) * (dk + 8) * 2 + 16 * 72 * 2 + 2 * LA_WARPS * 16 * sizeof(float);
  static bool configured[AF_MAX_DEVICES] = {};
  const int dev = af_current_device();
  if (dev < 0) return -1;
  if (!configured[dev]) {
    const size_t most = (size_t)(16 + LA_KEYS) * (LA_MAX_DK + 8) * 2 + 16 * 72 * 2 + 2 * LA_WARPS * 16 * sizeof(float);
    cudaError_t e = cudaFuncSetAttribute(attn_decode_latent_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)most);
    if (e != cudaSuccess) return af_fail((int)e, "af_attn_decode_latent: %s", cudaGetErrorString(e));
    configured[dev] = true;
  }
  af_launch(attn_decode_latent_kernel, dim3(n_splits, nkv * tiles, batch), dim3(LA_WARPS * 32), smem, stream,
            (const __nv_bfloat16*)q, q_stride, (const __nv_bfloat16*)kcache, page_table, max_pages, slots, lens, nq, nkv, dk,
            dv, scale, window, mask_kind, ring_rows, n_splits, part_o, part_ml);
  AF_CHECK_LAUNCH("af_attn_decode_latent");
}
