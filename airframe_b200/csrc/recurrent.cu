// Mixers that carry a state of fixed size from token to token instead of keys
// and values: matrix-valued states per head (linear attention with a decay per
// head; the generalized delta rule with a decay per key channel and a removal
// term) and vector-valued states (a gated recurrence whose gates read only the
// current token).  The state and everything that enters the recurrence is
// 32-bit in both precisions; the kernels read the projections as 32-bit rows.
//
// A state of one sequence, run and head is stored [value column][key channel]:
// the key channels of a column lie together, so that the lanes that share a
// column read and write whole 16-byte pieces.
#include "common.cuh"

// ---------------------------------------------------------------- what enters the delta rule

// From the packed projection row of a token: per head and key channel c
//   unit key   u = k / sqrt(sum_c k^2 + key_eps)
//   decay      w = exp(-decay_scale * sigmoid(w2 . tanh(w1 row) + w0))
//   removal    au = sigmoid(a + a_bias) * u
// written as float rows [token][3][heads * dk] (w, u, au).  One block per token, a warp per head.
__global__ void __launch_bounds__(128)
delta_prep_kernel(float* __restrict__ out, const float* __restrict__ proj, long long ld, int off_k, int off_a,
                  int off_w1, const float* __restrict__ a_bias, const float* __restrict__ w0,
                  const float* __restrict__ w2, int rank, int heads, int dk, float decay_scale, float key_eps) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float low[];                // tanh of the low-rank row
  const int t = blockIdx.x;
  const float* row = proj + (size_t)t * ld;
  for (int l = threadIdx.x; l < rank; l += blockDim.x) low[l] = tanhf(row[off_w1 + l]);
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
  const int n = heads * dk;
  float* o = out + (size_t)t * 3 * n;
  for (int h = warp; h < heads; h += nwarp) {
    float ss = 0.f;
    for (int c = lane; c < dk; c += 32) {
      const float kv = row[off_k + h * dk + c];
      ss += kv * kv;
    }
    ss = warp_sum(ss);
    const float nrm = sqrtf(ss + key_eps);
    for (int c = lane; c < dk; c += 32) {
      const int i = h * dk + c;
      float z = w0[i];
      const float* wr = w2 + (size_t)i * rank;
      for (int l = 0; l < rank; ++l) z += low[l] * wr[l];
      const float sig = 1.f / (1.f + expf(-z));
      const float u = row[off_k + i] / nrm;
      const float a = 1.f / (1.f + expf(-(row[off_a + i] + a_bias[i])));
      o[i] = expf(-decay_scale * sig);
      o[n + i] = u;
      o[2 * n + i] = a * u;
    }
  }
}

AF_EXPORT int af_delta_prep(float* out, const float* proj, long long ld, int off_k, int off_a, int off_w1,
                            const float* a_bias, const float* w0, const float* w2, int rank, int n_tokens, int heads,
                            int dk, float decay_scale, float key_eps, cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  AF_REQUIRE(n_tokens > 0 && heads > 0 && dk > 0 && rank > 0 && rank <= 8192, "af_delta_prep: bad sizes");
  af_launch(delta_prep_kernel, dim3(n_tokens), dim3(128), (size_t)rank * sizeof(float), stream, out, proj, ld, off_k,
            off_a, off_w1, a_bias, w0, w2, rank, heads, dk, decay_scale, key_eps);
  AF_CHECK_LAUNCH("af_delta_prep");
}

// ---------------------------------------------------------------- the scan over a matrix state

enum AfScanMode { AF_SCAN_DECAY = 0, AF_SCAN_DELTA = 1 };

// The vectors of a token and head that the scan reads (float rows; `*_ts` is the distance between
// tokens in elements; head h's piece starts h * dk (h * dv for v) behind the pointer):
//   DECAY:  S <- decay[h] S + k v^T                          o = S^T q     (q = `r`)
//   DELTA:  S <- diag(w) S - au (u^T S) + k v^T              o = S^T r     (both terms read the old S)
// With `silu` the r, k and v values go through x / (1 + exp(-x)) as they are read.
struct AfScanArgs {
  const float *r, *k, *v, *w, *u, *au;
  long long r_ts, k_ts, v_ts, w_ts, u_ts, au_ts;
  const float* decay;          // [heads] (DECAY)
  float* state;                // [slots][heads][dv][dk]
  float* out;                  // [tokens][heads * dv]
  long long out_ts;
  const int* seq_starts;       // [sequences + 1] first row of each sequence of the step
  const int* slots;            // [sequences] state slot, -1: a padding row (nothing read or written but zeros out)
  int heads, dk, dv;
  int lanes;                   // P: lanes that share a value column (a power of two); lane p holds key channels p R .. p R + R - 1
  int cols;                    // value columns of a block
  int chunk;                   // tokens staged in shared memory at a time
  int silu;
};

#define AF_SCAN_PREFETCH 24    // values a thread holds in registers for the chunk after the current one

// One block per (column tile, head, sequence); thread = (column, lane of the column).  The block walks
// the sequence's tokens in chunks: while it scans a chunk out of shared memory, the next chunk's vectors
// are on their way into registers.  Key channel c lives at (c / R) (R + 4) + c % R of a staged vector (four
// floats of padding per lane's run keep the 16-byte reads of a quarter warp in different banks).
template <int R, int MODE>
__global__ void __launch_bounds__(256)
state_scan_kernel(AfScanArgs a) {
  pdl_launch_dependents();
  extern __shared__ __align__(16) float smem[];
  const int P = a.lanes, CT = a.cols, CH = a.chunk, dk = a.dk, dv = a.dv;
  const int NV = MODE == AF_SCAN_DELTA ? 5 : 2;             // staged key-sized vectors: r, k (, w, u, au)
  const int dkp = P * (R + 4);
  const int tok_floats = NV * dkp + CT;                     // a token's staged floats: the vectors, then its v tile
  const int buf_floats = CH * tok_floats;
  const int tid = threadIdx.x, nthr = blockDim.x;
  const int part = tid % P, col = tid / P;
  const int h = blockIdx.y, b = blockIdx.z;
  const int j0 = blockIdx.x * CT, j = j0 + col;
  const bool col_on = j < dv;
  // a token's values in the order they are fetched: NV key vectors of dk, then CT values of v
  const int tok_vals = NV * dk + CT;
  const int first = a.seq_starts[b], last = a.seq_starts[b + 1];
  const int slot = a.slots[b];
  pdl_wait();
  if (slot < 0) {
    for (int t = first + tid / CT; t < last; t += nthr / CT)
      if (j0 + tid % CT < dv) a.out[(size_t)t * a.out_ts + h * dv + j0 + tid % CT] = 0.f;
    return;
  }
  for (int i = tid; i < 2 * buf_floats; i += nthr) smem[i] = 0.f;        // (the padding stays zero for good)
  // the state's piece of this thread
  float S[R];
  float* st = a.state + (((size_t)slot * a.heads + h) * dv + (col_on ? j : 0)) * dk + part * R;
#pragma unroll
  for (int i = 0; i < R; ++i) S[i] = (col_on && part * R + i < dk) ? st[i] : 0.f;
  const float dec = MODE == AF_SCAN_DECAY ? a.decay[h] : 0.f;

  float pf[AF_SCAN_PREFETCH];
  auto fetch = [&](int t0, int n) {                          // tokens t0 .. t0 + n - 1 into registers
#pragma unroll
    for (int e = 0; e < AF_SCAN_PREFETCH; ++e) {
      const int idx = tid + e * nthr;
      float val = 0.f;
      if (idx < n * tok_vals) {
        const int tt = idx / tok_vals, x = idx - tt * tok_vals;
        const size_t t = (size_t)(t0 + tt);
        if (x < NV * dk) {
          const int vec = x / dk, c = x - vec * dk;
          const float* p = vec == 0 ? a.r + t * a.r_ts : vec == 1 ? a.k + t * a.k_ts
                         : vec == 2 ? a.w + t * a.w_ts : vec == 3 ? a.u + t * a.u_ts : a.au + t * a.au_ts;
          val = p[h * dk + c];
          if (a.silu) val = val / (1.f + expf(-val));
        } else {
          const int jj = j0 + x - NV * dk;
          if (jj < dv) {
            val = a.v[t * a.v_ts + h * dv + jj];
            if (a.silu) val = val / (1.f + expf(-val));
          }
        }
      }
      pf[e] = val;
    }
  };
  auto stage = [&](float* buf, int n) {                      // registers into a shared-memory buffer
#pragma unroll
    for (int e = 0; e < AF_SCAN_PREFETCH; ++e) {
      const int idx = tid + e * nthr;
      if (idx < n * tok_vals) {
        const int tt = idx / tok_vals, x = idx - tt * tok_vals;
        int at;
        if (x < NV * dk) {
          const int vec = x / dk, c = x - vec * dk;
          at = vec * dkp + (c / R) * (R + 4) + c % R;
        } else {
          at = NV * dkp + x - NV * dk;
        }
        buf[tt * tok_floats + at] = pf[e];
      }
    }
  };

  int t0 = first;
  int n = min(CH, last - t0);
  fetch(t0, n);
  __syncthreads();                                           // (the zeroing is done)
  int which = 0;
  while (t0 < last) {
    float* buf = smem + which * buf_floats;
    stage(buf, n);
    __syncthreads();
    const int t1 = t0 + n;
    const int n1 = min(CH, last - t1);
    if (n1 > 0) fetch(t1, n1);                               // under the scan of this chunk
    for (int tt = 0; tt < n; ++tt) {
      const float* tk = buf + tt * tok_floats + part * (R + 4);
      const float vj = buf[tt * tok_floats + NV * dkp + col];
      float rv[R], kv[R];
#pragma unroll
      for (int i = 0; i < R; i += 4) {
        *reinterpret_cast<float4*>(rv + i) = *reinterpret_cast<const float4*>(tk + i);
        *reinterpret_cast<float4*>(kv + i) = *reinterpret_cast<const float4*>(tk + dkp + i);
      }
      if (MODE == AF_SCAN_DELTA) {
        float wv[R], uv[R], av[R];
#pragma unroll
        for (int i = 0; i < R; i += 4) {
          *reinterpret_cast<float4*>(wv + i) = *reinterpret_cast<const float4*>(tk + 2 * dkp + i);
          *reinterpret_cast<float4*>(uv + i) = *reinterpret_cast<const float4*>(tk + 3 * dkp + i);
          *reinterpret_cast<float4*>(av + i) = *reinterpret_cast<const float4*>(tk + 4 * dkp + i);
        }
        float d0 = 0.f, d1 = 0.f;
#pragma unroll
        for (int i = 0; i < R; i += 2) {
          d0 += uv[i] * S[i];
          d1 += uv[i + 1] * S[i + 1];
        }
        float dot = d0 + d1;
        for (int o = 1; o < P; o <<= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
#pragma unroll
        for (int i = 0; i < R; ++i) S[i] = wv[i] * S[i] - av[i] * dot + kv[i] * vj;
      } else {
#pragma unroll
        for (int i = 0; i < R; ++i) S[i] = dec * S[i] + kv[i] * vj;
      }
      float o0 = 0.f, o1 = 0.f;
#pragma unroll
      for (int i = 0; i < R; i += 2) {
        o0 += rv[i] * S[i];
        o1 += rv[i + 1] * S[i + 1];
      }
      float o = o0 + o1;
      for (int s = 1; s < P; s <<= 1) o += __shfl_xor_sync(0xffffffffu, o, s);
      if (part == 0 && col_on) a.out[(size_t)(t0 + tt) * a.out_ts + h * dv + j] = o;
    }
    t0 = t1;
    n = n1;
    which ^= 1;
  }
  if (col_on) {
#pragma unroll
    for (int i = 0; i < R; ++i)
      if (part * R + i < dk) st[i] = S[i];
  }
}

template <int R>
static int launch_scan(const AfScanArgs& a, int mode, dim3 grid, int threads, size_t smem, cudaStream_t stream) {
  static bool raised[2][AF_MAX_DEVICES];
  auto k0 = state_scan_kernel<R, AF_SCAN_DECAY>;
  auto k1 = state_scan_kernel<R, AF_SCAN_DELTA>;
  if (smem > 48 * 1024) {
    const int dev = af_current_device();
    if (dev < 0) return -1;
    if (af_first_on_device(raised[mode], dev)) {
      cudaError_t e = cudaFuncSetAttribute(mode == AF_SCAN_DELTA ? k1 : k0, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           96 * 1024);
      if (e != cudaSuccess) return af_fail((int)e, "af_state_scan: %s", cudaGetErrorString(e));
    }
  }
  if (mode == AF_SCAN_DELTA) af_launch(k1, grid, dim3(threads), smem, stream, a);
  else af_launch(k0, grid, dim3(threads), smem, stream, a);
  AF_CHECK_LAUNCH("af_state_scan");
}

// The cut of a scan: R key channels a lane, P lanes a column, CT columns a block, CH tokens a chunk.
static void scan_cut(int mode, int dk, int dv, int* R, int* P, int* CT, int* CH) {
  int r = 4;
  while (r < 32 && (dk + r - 1) / r > 8) r *= 2;            // up to eight lanes a column while a lane holds up to 32
  int p = 1;
  while (p * r < dk && p < 32) p *= 2;
  int ct = 128 / p;                                          // 128 threads a block
  while (ct > 4 && ct / 2 >= dv && (ct / 2) * p >= 32) ct /= 2;   // (no wider than the state's columns need; whole warps)
  const int nv = mode == AF_SCAN_DELTA ? 5 : 2;
  const int tok_vals = nv * dk + ct, tok_floats = nv * p * (r + 4) + ct;
  int ch = 16;
  while (ch > 1 && (ch * tok_vals > AF_SCAN_PREFETCH * ct * p || 2 * ch * tok_floats * 4 > 96 * 1024)) ch /= 2;
  *R = r, *P = p, *CT = ct, *CH = ch;
}

AF_EXPORT int af_state_scan(int mode, const float* r, long long r_ts, const float* k, long long k_ts, const float* v,
                            long long v_ts, const float* w, long long w_ts, const float* u, long long u_ts,
                            const float* au, long long au_ts, const float* decay, float* state, float* out,
                            long long out_ts, const int* seq_starts, const int* slots, int n_seqs, int heads, int dk,
                            int dv, int silu, cudaStream_t stream) {
  if (n_seqs == 0) return 0;
  AF_REQUIRE(mode == AF_SCAN_DECAY || mode == AF_SCAN_DELTA, "af_state_scan: mode %d", mode);
  AF_REQUIRE(n_seqs > 0 && heads > 0 && dk > 0 && dv > 0 && dk <= 1024, "af_state_scan: bad sizes (key size up to 1024)");
  AF_REQUIRE(n_seqs < 65536 && heads < 65536, "af_state_scan: too many sequences or heads for one grid");
  AfScanArgs a;
  a.r = r, a.k = k, a.v = v, a.w = w, a.u = u, a.au = au;
  a.r_ts = r_ts, a.k_ts = k_ts, a.v_ts = v_ts, a.w_ts = w_ts, a.u_ts = u_ts, a.au_ts = au_ts;
  a.decay = decay, a.state = state, a.out = out, a.out_ts = out_ts, a.seq_starts = seq_starts, a.slots = slots;
  a.heads = heads, a.dk = dk, a.dv = dv, a.silu = silu;
  int R, P, CT, CH;
  scan_cut(mode, dk, dv, &R, &P, &CT, &CH);
  AF_REQUIRE(P * R >= dk, "af_state_scan: key size %d does not fit %d lanes of %d", dk, P, R);
  const int nv = mode == AF_SCAN_DELTA ? 5 : 2;
  AF_REQUIRE(CH * (nv * dk + CT) <= AF_SCAN_PREFETCH * CT * P, "af_state_scan: a token of %d values is too long to stage",
             nv * dk + CT);
  a.lanes = P, a.cols = CT, a.chunk = CH;
  const size_t smem = (size_t)2 * CH * (nv * P * (R + 4) + CT) * sizeof(float);
  const dim3 grid((dv + CT - 1) / CT, heads, n_seqs);
  switch (R) {
    case 4: return launch_scan<4>(a, mode, grid, CT * P, smem, stream);
    case 8: return launch_scan<8>(a, mode, grid, CT * P, smem, stream);
    case 16: return launch_scan<16>(a, mode, grid, CT * P, smem, stream);
    default: return launch_scan<32>(a, mode, grid, CT * P, smem, stream);
  }
}

// ---------------------------------------------------------------- the output of a state mixer

// y[t][i] = o[t][i] * rsqrt(mean over i's group of o^2 + eps) * w[i] * sigmoid(gate[t][i]): a norm over groups
// of `group` values (a head, or the whole row) with a plain weight, times a gate.  One block per token.
template <typename TY>
__global__ void __launch_bounds__(256)
gated_group_norm_kernel(TY* __restrict__ y, const float* __restrict__ o, const float* __restrict__ w,
                        const float* __restrict__ gate, long long gate_ts, int n, int group, float eps) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float scratch[33];
  const int t = blockIdx.x;
  const float* orow = o + (size_t)t * n;
  const float* grow = gate + (size_t)t * gate_ts;
  TY* yrow = y + (size_t)t * n;
  if (group == n) {
    float ss = 0.f;
    for (int i = threadIdx.x; i < n; i += blockDim.x) ss += orow[i] * orow[i];
    ss = block_sum(ss, scratch);
    const float inv = rsqrtf(ss / (float)n + eps);
    for (int i = threadIdx.x; i < n; i += blockDim.x)
      yrow[i] = from_f32<TY>(orow[i] * inv * w[i] * (1.f / (1.f + expf(-grow[i]))));
    return;
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
  for (int g = warp; g < n / group; g += nwarp) {
    float ss = 0.f;
    for (int c = lane; c < group; c += 32) ss += orow[g * group + c] * orow[g * group + c];
    ss = warp_sum(ss);
    const float inv = rsqrtf(ss / (float)group + eps);
    for (int c = lane; c < group; c += 32) {
      const int i = g * group + c;
      yrow[i] = from_f32<TY>(orow[i] * inv * w[i] * (1.f / (1.f + expf(-grow[i]))));
    }
  }
}

AF_EXPORT int af_gated_group_norm(void* y, int y_dtype, const float* o, const float* w, const float* gate,
                                  long long gate_ts, int n_tokens, int n, int group, float eps, cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  AF_REQUIRE(n_tokens > 0 && n > 0 && group > 0 && n % group == 0, "af_gated_group_norm: %d values in groups of %d", n, group);
  AF_DISPATCH_DTYPE(y_dtype, TY, af_launch(gated_group_norm_kernel<TY>, dim3(n_tokens), dim3(256), 0, stream, (TY*)y, o, w,
                                           gate, gate_ts, n, group, eps));
  AF_CHECK_LAUNCH("af_gated_group_norm");
}

// ---------------------------------------------------------------- a gated recurrence over a vector state

// Per channel: z = sigmoid(pz + bz), c = px + bx, candidate = c + 1/2 where c >= 0 and sigmoid(c) below,
// S <- (1 - z) S + z candidate, y = S * silu(pg).  pz, px, pg are sections of the packed projection row.
// One thread per (sequence, channel); the loads of four tokens are issued before the chain goes on.
template <typename TY>
__global__ void __launch_bounds__(128)
gated_scan_kernel(TY* __restrict__ y, const float* __restrict__ proj, long long ld, int off_z, int off_x, int off_g,
                  const float* __restrict__ bz, const float* __restrict__ bx, float* __restrict__ state,
                  const int* __restrict__ seq_starts, const int* __restrict__ slots, int width) {
  pdl_launch_dependents();
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  const int b = blockIdx.y;
  if (c >= width) return;
  const int first = seq_starts[b], last = seq_starts[b + 1];
  const int slot = slots[b];
  const float zb = bz[c], xb = bx[c];
  pdl_wait();
  if (slot < 0) {
    for (int t = first; t < last; ++t) y[(size_t)t * width + c] = from_f32<TY>(0.f);
    return;
  }
  float S = state[(size_t)slot * width + c];
  for (int t = first; t < last; t += 4) {
    float pz[4], px[4], pg[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const bool on = t + e < last;
      const float* row = proj + (size_t)(t + e) * ld + c;
      pz[e] = on ? row[off_z] : 0.f;
      px[e] = on ? row[off_x] : 0.f;
      pg[e] = on ? row[off_g] : 0.f;
    }
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      if (t + e >= last) break;
      const float z = 1.f / (1.f + expf(-(pz[e] + zb)));
      const float u = px[e] + xb;
      const float cand = u >= 0.f ? u + 0.5f : 1.f / (1.f + expf(-u));
      S = (1.f - z) * S + z * cand;
      const float g = pg[e];
      y[(size_t)(t + e) * width + c] = from_f32<TY>(S * (g / (1.f + expf(-g))));
    }
  }
  state[(size_t)slot * width + c] = S;
}

AF_EXPORT int af_gated_scan(void* y, int y_dtype, const float* proj, long long ld, int off_z, int off_x, int off_g,
                            const float* bz, const float* bx, float* state, const int* seq_starts, const int* slots,
                            int n_seqs, int width, cudaStream_t stream) {
  if (n_seqs == 0) return 0;
  AF_REQUIRE(n_seqs > 0 && n_seqs < 65536 && width > 0, "af_gated_scan: bad sizes");
  AF_DISPATCH_DTYPE(y_dtype, TY, af_launch(gated_scan_kernel<TY>, dim3((width + 127) / 128, n_seqs), dim3(128), 0, stream,
                                           (TY*)y, proj, ld, off_z, off_x, off_g, bz, bx, state, seq_starts, slots, width));
  AF_CHECK_LAUNCH("af_gated_scan");
}
