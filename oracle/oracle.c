/*
 * CPU restatement of the GrainGEMM hot path.  TEST INFRASTRUCTURE ONLY.
 *
 * This file is the parity oracle for the CUDA library: tests, the smoke check
 * and the benchmark's cpu_baseline / reference arm may call it; the product
 * (the Python package and the C-ABI library) never does.
 *
 * Every function restates, in plain C, the arithmetic of one piece of the
 * reference (paths are relative to the reference project):
 *
 *   oracle_int8_gemm / oracle_group_partials
 *       src/grain_gemm/kernels/triton.py:28-51  (per-group INT32 dot, FP32
 *       scale product rounded once, fused multiply-add into an FP32 total
 *       that starts at 0, one cast at the end)
 *   oracle_route
 *       src/grain_gemm/kernels/moe.py:48-99,102-171,222-291  (keys with the
 *       range check at the ids' own width, stable sort with the invalid tail,
 *       inverse, counts, offsets, statistics)
 *   oracle_swiglu_quantize
 *   oracle_quantize_rows
 *       src/grain_gemm/kernels/moe.py:321-328,564-601  (SwiGLU on the rounded
 *       gate/up values, per row and 256-channel group amax -> scale ->
 *       nearest-even quantisation clipped to +-127, no FMA contraction)
 *   oracle_ragged_gemm
 *       src/grain_gemm/kernels/moe.py:359-393  (one grouped GEMM per sorted
 *       slot, optional gather of the source row by order[slot] / R)
 *   oracle_combine
 *       src/grain_gemm/kernels/moe.py:634-653  (FP32 weighted sum over the
 *       top-k slots of a token in slot order, product and sum unfused)
 *
 * Parity status: pinned.  tests/test_oracle.py checks these functions against
 * fixtures produced by the reference's own CPU code and by the reference's
 * Triton kernels run under Triton's CPU interpreter (tests/golden/).
 * Known limit: expf here is the host C library's, the reference calls CUDA
 * libdevice; the two may differ in the last bit, which can move a quantised
 * activation by one step on a rounding boundary.
 *
 * Build: see oracle/Makefile (gcc -O3 -mavx2 -mfma -fopenmp -ffp-contract=off).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

int oracle_abi_version(void) { return 2; }

/* silu(v) = v / (1 + expf(-v)) for n values, with the host C library's expf. */
void oracle_silu(const float* in, float* out, int64_t n) {
  for (int64_t i = 0; i < n; ++i) out[i] = in[i] / (1.0f + expf(-in[i]));
}

int oracle_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

/* ---- rounding helpers (round-to-nearest-even, like torch's .to()) -------- */

static inline uint32_t f2u(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }
static inline float u2f(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }

static inline float round_bf16(float f) {
  uint32_t u = f2u(f);
  if ((u & 0x7fffffffu) > 0x7f800000u) return u2f(u | 0x00400000u); /* NaN */
  uint32_t bias = 0x7fffu + ((u >> 16) & 1u);
  u += bias;
  return u2f(u & 0xffff0000u);
}

static inline float round_f16(float f) {
  _Float16 h = (_Float16)f; /* gcc converts with RN-even */
  return (float)h;
}

/* out_kind: 0 = fp32 (identity), 1 = bf16, 2 = fp16; result is the rounded
 * value held in a float. */
static inline float round_out(float f, int out_kind) {
  return out_kind == 1 ? round_bf16(f) : out_kind == 2 ? round_f16(f) : f;
}

void oracle_round(const float* in, float* out, int64_t n, int out_kind) {
  for (int64_t i = 0; i < n; ++i) out[i] = round_out(in[i], out_kind);
}

/* ---- grouped GEMM --------------------------------------------------------- */

static inline int32_t dot_i8(const int8_t* a, const int8_t* b, int n) {
  int32_t s = 0;
  for (int i = 0; i < n; ++i) s += (int32_t)a[i] * (int32_t)b[i];
  return s;
}

/* Packs a strided int8 matrix [rows, cols] into a contiguous row-major copy. */
static int8_t* pack_rows(const int8_t* src, int64_t rows, int64_t cols,
                         int64_t stride_r, int64_t stride_c) {
  int8_t* dst = (int8_t*)malloc((size_t)(rows * cols > 0 ? rows * cols : 1));
  if (!dst) return NULL;
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < rows; ++r)
    for (int64_t c = 0; c < cols; ++c)
      dst[r * cols + c] = src[r * stride_r + c * stride_c];
  return dst;
}

/*
 * C[m,n] = cast( sum over groups in order:
 *                fmaf((float)dot_i32(A[m,g], B[g,n]), sa[m,g]*sb[g,n], total) )
 * A is [M,K] with element strides (a_sm, a_sk); B is [K,N] with (b_sk, b_sn);
 * scale_a [M,Q] (sa_sm, sa_sg); scale_b [Q,N] (sb_sg, sb_sn); Q = ceil(K/G).
 * A partial last group contributes only its present elements.
 * out is FP32 [M,N] row-major holding the value rounded to out_kind.
 * partials, when not NULL, receives the INT32 group dots as [M,N,Q].
 */
int oracle_int8_gemm(const int8_t* a, const int8_t* b, const float* sa, const float* sb,
                     float* out, int32_t* partials,
                     int64_t M, int64_t N, int64_t K,
                     int64_t a_sm, int64_t a_sk, int64_t b_sk, int64_t b_sn,
                     int64_t sa_sm, int64_t sa_sg, int64_t sb_sg, int64_t sb_sn,
                     int G, int out_kind) {
  if (M < 0 || N < 0 || K < 0 || G <= 0) return 1;
  if (M == 0 || N == 0) return 0;
  int64_t Q = (K + G - 1) / G;
  int8_t* ap = pack_rows(a, M, K, a_sm, a_sk);
  int8_t* bp = pack_rows(b, N, K, b_sn, b_sk); /* B^T: [N,K] */
  if (!ap || !bp) { free(ap); free(bp); return 2; }
#pragma omp parallel for schedule(dynamic, 1) collapse(2)
  for (int64_t m = 0; m < M; ++m) {
    for (int64_t nb = 0; nb < N; nb += 64) {
      int64_t ne = nb + 64 < N ? nb + 64 : N;
      for (int64_t n = nb; n < ne; ++n) {
        float total = 0.0f;
        for (int64_t g = 0; g < Q; ++g) {
          int64_t k0 = g * G;
          int len = (int)(K - k0 < G ? K - k0 : G);
          int32_t p = dot_i8(ap + m * K + k0, bp + n * K + k0, len);
          if (partials) partials[(m * N + n) * Q + g] = p;
          float scale = sa[m * sa_sm + g * sa_sg] * sb[g * sb_sg + n * sb_sn];
          total = fmaf((float)p, scale, total);
        }
        out[m * N + n] = round_out(total, out_kind);
      }
    }
  }
  free(ap);
  free(bp);
  return 0;
}

/* ---- routing --------------------------------------------------------------- */

/*
 * ids: [T*R] int32 (ids_is_i64 == 0) or int64; mask: [T] bytes or NULL.
 * effective_ids: same width as ids, key = id if the token is enabled and
 * 0 <= id < E (tested at the ids' width), else E.
 * order [S] int64: stable sort of assignments by key (invalid tail included);
 * inverse [S] int32: sorted slot or -1; counts [E]; offsets [E+1];
 * statistics [3] = (enabled-but-out-of-range count, max count, valid total).
 */
int oracle_route(const void* ids, int ids_is_i64, const uint8_t* mask,
                 int64_t T, int64_t R, int64_t E,
                 void* effective_ids, int64_t* order, int32_t* inverse,
                 int32_t* counts, int32_t* offsets, int32_t* statistics) {
  int64_t S = T * R;
  int64_t* keys = (int64_t*)malloc(sizeof(int64_t) * (size_t)(S > 0 ? S : 1));
  int64_t* fill = (int64_t*)calloc((size_t)(E + 2), sizeof(int64_t));
  if (!keys || !fill) { free(keys); free(fill); return 2; }
  int32_t invalid = 0;
  for (int64_t e = 0; e < E; ++e) counts[e] = 0;
  for (int64_t s = 0; s < S; ++s) {
    int64_t id = ids_is_i64 ? ((const int64_t*)ids)[s] : (int64_t)((const int32_t*)ids)[s];
    int enabled = mask ? mask[s / R] != 0 : 1;
    int in_range = id >= 0 && id < E;
    int64_t key = (enabled && in_range) ? id : E;
    if (enabled && !in_range) ++invalid;
    keys[s] = key;
    if (ids_is_i64) ((int64_t*)effective_ids)[s] = key;
    else ((int32_t*)effective_ids)[s] = (int32_t)key;
    if (key < E) ++counts[key];
    ++fill[key + 1];
  }
  offsets[0] = 0;
  int32_t maximum = 0;
  for (int64_t e = 0; e < E; ++e) {
    offsets[e + 1] = offsets[e] + counts[e];
    if (counts[e] > maximum) maximum = counts[e];
  }
  for (int64_t e = 0; e <= E; ++e) fill[e + 1] += fill[e]; /* fill[e] = start of key e */
  for (int64_t s = 0; s < S; ++s) {
    int64_t slot = fill[keys[s]]++;
    order[slot] = s;
    inverse[s] = keys[s] < E ? (int32_t)slot : -1;
  }
  statistics[0] = invalid;
  statistics[1] = maximum;
  statistics[2] = offsets[E];
  free(keys);
  free(fill);
  return 0;
}

/* ---- SwiGLU + G256 requantisation ------------------------------------------ */

/*
 * gate_up: [rows, 2I] FP32 holding values already rounded to the output dtype.
 * valid_rows: rows at index >= valid_rows are treated as invalid (q = 0,
 * scale = 1e-12f/127).  interleaved: gate = column 2j, up = column 2j+1,
 * otherwise gate = column j, up = column I + j.
 * q: [rows, I] int8; s: [rows, I/256] FP32.
 */
/*
 * silu_table (optional): 65536 values of silu indexed by the gate's 16-bit pattern in the
 * type named by table_kind (1 = bf16, 2 = fp16).  The gate values handed in are already
 * rounded to that type, so the lookup is exact.  With a table the function evaluates
 * silu by lookup instead of gate / (1 + expf(-gate)); tests pass the table the CUDA library
 * computes with the same formula on the GPU, which removes the one place where host and
 * device arithmetic (expf) can differ in the last bit.
 */
static inline uint32_t gate_bits(float gate, int table_kind) {
  if (table_kind == 1) return f2u(gate) >> 16;
  _Float16 h = (_Float16)gate;
  uint16_t bits;
  memcpy(&bits, &h, 2);
  return bits;
}

int oracle_swiglu_quantize(const float* gate_up, int64_t rows, int64_t valid_rows,
                           int64_t I, int interleaved, int8_t* q, float* s,
                           const float* silu_table, int table_kind) {
  if (I % 256) return 1;
  if (silu_table && table_kind != 1 && table_kind != 2) return 1;
  int64_t groups = I / 256;
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < rows; ++r) {
    float h[256];
    for (int64_t g = 0; g < groups; ++g) {
      int8_t* qr = q + r * I + g * 256;
      if (r >= valid_rows) {
        memset(qr, 0, 256);
        s[r * groups + g] = 1.0e-12f / 127.0f;
        continue;
      }
      float amax = 0.0f;
      for (int j = 0; j < 256; ++j) {
        int64_t c = g * 256 + j;
        float gate = gate_up[r * 2 * I + (interleaved ? 2 * c : c)];
        float up = gate_up[r * 2 * I + (interleaved ? 2 * c + 1 : I + c)];
        float silu;
        if (silu_table) {
          silu = silu_table[gate_bits(gate, table_kind)];
        } else {
          float denom = 1.0f + expf(-gate);
          silu = gate / denom;
        }
        h[j] = silu * up;
        float v = fabsf(h[j]);
        if (v > amax || v != v) amax = v;
      }
      float m = amax > 1.0e-12f ? amax : 1.0e-12f;
      float scale = m / 127.0f;
      s[r * groups + g] = scale;
      for (int j = 0; j < 256; ++j) {
        float v = nearbyintf(h[j] / scale);
        v = v < -127.0f ? -127.0f : v > 127.0f ? 127.0f : v;
        qr[j] = (int8_t)v;
      }
    }
  }
  return 0;
}

/* ---- entry quantiser -------------------------------------------------------- */

/*
 * Symmetric per-row, per-K-group quantisation of floating rows, restating
 * _symmetric_quantize_row_block / quantize_rows (src/grain_gemm/kernels/moe.py:321-356):
 *   scale = div_rn(max(amax, 1e-12), 127);  q = clamp(nearbyint(div_rn(v, scale)), -127, 127).
 * x: [rows, width] FP32 (the caller converts BF16/FP16 exactly); q: [rows, width] int8;
 * s: [rows, width / group] FP32.
 */
int oracle_quantize_rows(const float* x, int64_t rows, int64_t width, int64_t group, int8_t* q,
                         float* s) {
  if (group <= 0 || width % group) return 1;
  int64_t groups = width / group;
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < rows; ++r) {
    for (int64_t g = 0; g < groups; ++g) {
      const float* v = x + r * width + g * group;
      float amax = 0.0f;
      for (int64_t j = 0; j < group; ++j) {
        float a = fabsf(v[j]);
        if (a > amax || a != a) amax = a;
      }
      float m = amax > 1.0e-12f ? amax : 1.0e-12f;
      float scale = m / 127.0f;
      s[r * groups + g] = scale;
      for (int64_t j = 0; j < group; ++j) {
        float t = nearbyintf(v[j] / scale);
        t = t < -127.0f ? -127.0f : t > 127.0f ? 127.0f : t;
        q[r * width + g * group + j] = (int8_t)t;
      }
    }
  }
  return 0;
}

/* ---- ragged (per sorted slot) grouped GEMM --------------------------------- */

/*
 * For each sorted slot < offsets[E] belonging to expert e:
 *   source row = gather ? order[slot] / R : slot
 *   out[slot, :] = grouped GEMM row of A[source] against W[e] (Linear [N,K]
 *   contiguous) with scale rows sa[source, K/256] and sb[e, K/256, N], G = 256.
 * Slots at and beyond offsets[E] are left untouched.
 */
int oracle_ragged_gemm(const int8_t* a, const float* sa, const int8_t* w, const float* sb,
                       const int64_t* order, const int32_t* offsets,
                       float* out, int64_t E, int64_t N, int64_t K, int64_t R,
                       int gather, int out_kind) {
  if (K % 256) return 1;
  int64_t Q = K / 256;
#pragma omp parallel for schedule(dynamic, 1)
  for (int64_t e = 0; e < E; ++e) {
    for (int64_t slot = offsets[e]; slot < offsets[e + 1]; ++slot) {
      int64_t src = gather ? order[slot] / R : slot;
      const int8_t* ar = a + src * K;
      for (int64_t n = 0; n < N; ++n) {
        const int8_t* wr = w + (e * N + n) * K;
        float total = 0.0f;
        for (int64_t g = 0; g < Q; ++g) {
          int32_t p = dot_i8(ar + g * 256, wr + g * 256, 256);
          float scale = sa[src * Q + g] * sb[(e * Q + g) * N + n];
          total = fmaf((float)p, scale, total);
        }
        out[slot * N + n] = round_out(total, out_kind);
      }
    }
  }
  return 0;
}

/* ---- top-k weighted combine ------------------------------------------------- */

/*
 * out[t,:] = cast( sum_{r in slot order, inverse[t*R+r] >= 0}
 *                  expert_out[inverse[t*R+r], :] * weights[t,r] )
 * expert_out holds FP32 copies of the rounded expert outputs; the product is
 * rounded to FP32 before the add (no FMA).
 */
int oracle_combine(const float* expert_out, const float* weights, const int32_t* inverse,
                   float* out, int64_t T, int64_t R, int64_t H, int out_kind) {
#pragma omp parallel for schedule(static)
  for (int64_t t = 0; t < T; ++t) {
    for (int64_t h = 0; h < H; ++h) {
      float total = 0.0f;
      for (int64_t r = 0; r < R; ++r) {
        int32_t slot = inverse[t * R + r];
        if (slot < 0) continue;
        float product = expert_out[(int64_t)slot * H + h] * weights[t * R + r];
        total = total + product;
      }
      out[t * H + h] = round_out(total, out_kind);
    }
  }
  return 0;
}

/* Element-wise exact fused multiply-add, used by the fixture generator to give
 * Triton's CPU interpreter a true FMA. */
void oracle_fmaf(const float* x, const float* y, const float* z, float* out, int64_t n) {
  for (int64_t i = 0; i < n; ++i) out[i] = fmaf(x[i], y[i], z[i]);
}
