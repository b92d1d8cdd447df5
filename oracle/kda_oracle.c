/*
 * CPU oracle for the Kimi Delta Attention (KDA) prefill `flash_kda.fwd`.
 *
 * TEST INFRASTRUCTURE ONLY.  Nothing in the shipped package may call into this
 * file; it exists so that tests, the smoke check and the benchmark's CPU
 * baseline leg have something independent to compare the CUDA path with.
 *
 * Three restatements live here, all for head dimension K = V = 128:
 *
 *   kda_oracle_recurrence   the per-token definition of the operator, in fp64.
 *                           Follows the gold construction the reference's own
 *                           accuracy tests use (tests/test_fwd.py:71-104: gate
 *                           and beta activations in fp64, then a token-by-token
 *                           delta-rule recurrence) and the state orientation of
 *                           tests/torch_ref.py:228-239 (state stored [V][K]).
 *
 *   kda_oracle_chunk16      the reference's chunked algorithm with every bf16
 *                           rounding point, restated from tests/torch_ref.py
 *                           (:62-78 L2 norm, :87-122 16x16 inverse, :129-247
 *                           main loop).  Two substitutions, because the
 *                           original needs a GPU: the MUFU `tanh.approx` based
 *                           sigmoid (:7-38) becomes tanhf(x/2)/2+1/2, and the
 *                           tensor-core products become fp32 dot products of
 *                           the (exact) bf16 operands.  Parity of this port is
 *                           pinned by tests/golden/ vectors that were produced
 *                           by importing tests/torch_ref.py itself.
 *
 *   kda_oracle_chunk_operands
 *                           fp64 values of the per-chunk operands of the
 *                           chunk-32 WY formulation the CUDA path uses (decayed
 *                           keys/queries, the triangular inverse applied to keys
 *                           and values, the intra-chunk q.k matrix, the chunk
 *                           decay).  Used to check the prepare kernel alone.
 *
 * Build: gcc -O3 -fopenmp -fPIC -shared (see oracle/build_oracle.py).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define D 128
#define LOG2E 1.4426950408889634

enum { STATE_NONE = 0, STATE_BF16 = 1, STATE_F32 = 2 };

/* ---------------------------------------------------------------- bf16 ---- */

static inline float bf2f(uint16_t b) {
  uint32_t u = ((uint32_t)b) << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}

/* round-to-nearest-even, the conversion torch and the GPU both use */
static inline uint16_t f2bf(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x40); /* NaN */
  uint32_t lsb = (u >> 16) & 1u;
  u += 0x7fffu + lsb;
  return (uint16_t)(u >> 16);
}

static inline float rbf(float f) { return bf2f(f2bf(f)); }

/* tests/torch_ref.py:47-52 : exp2 in fp32 with subnormal results flushed */
static inline float ex2_ftz(float x) {
  float r = exp2f(x);
  if (fabsf(r) < 1.17549435e-38f) r = 0.0f;
  return r;
}

/* tests/torch_ref.py:11-20 with tanh.approx replaced by tanhf */
static inline float sigmoid_tanh(float x) { return tanhf(x * 0.5f) * 0.5f + 0.5f; }

/* tests/torch_ref.py:55-59 : fma evaluated in fp64, rounded once to fp32 */
static inline float fma_via_f64(float c, float a, float b) {
  return (float)((double)c + (double)a * (double)b);
}

static int resolve_threads(int nthreads) {
#ifdef _OPENMP
  if (nthreads <= 0) nthreads = omp_get_max_threads();
  return nthreads;
#else
  (void)nthreads;
  return 1;
#endif
}

int kda_oracle_max_threads(void) { return resolve_threads(0); }

/* ------------------------------------------------ per-token fp64 oracle ---- */

/*
 * q,k,v,g : bf16 bit patterns, [T_total][H][128]
 * beta    : bf16 bit patterns, [T_total][H] (logits)
 * A_log   : fp32 [H];  dt_bias : fp32 [H][128]
 * init    : [N][H][128 (v)][128 (k)] bf16 or fp32, or NULL
 * cu      : int64 [N+1] sequence boundaries in tokens
 * head_lo/head_hi, seq_lo/seq_hi : sub-range of chains to evaluate (others untouched)
 * out_f64 : [T_total][H][128] doubles (only rows of evaluated chains written)
 * fin_f64 : [N][H][128][128] doubles, may be NULL
 */
int kda_oracle_recurrence(const uint16_t* q, const uint16_t* k, const uint16_t* v,
                          const uint16_t* g, const uint16_t* beta, const float* A_log,
                          const float* dt_bias, double scale, double lower_bound,
                          const void* init, int init_dtype, const int64_t* cu, int64_t N,
                          int64_t H, int64_t seq_lo, int64_t seq_hi, int64_t head_lo,
                          int64_t head_hi, double* out_f64, double* fin_f64, int nthreads) {
  if (!q || !k || !v || !g || !beta || !A_log || !dt_bias || !cu || !out_f64) return -1;
  int64_t nseq = seq_hi - seq_lo, nhead = head_hi - head_lo;
  if (nseq <= 0 || nhead <= 0) return 0;
  nthreads = resolve_threads(nthreads);
  int err = 0;
#pragma omp parallel for num_threads(nthreads) schedule(dynamic, 1)
  for (int64_t job = 0; job < nseq * nhead; ++job) {
    int64_t n = seq_lo + job / nhead, h = head_lo + job % nhead;
    double* S = (double*)malloc(sizeof(double) * D * D); /* S[kk][vv] */
    if (!S) { err = -2; continue; }
    for (int kk = 0; kk < D; ++kk)
      for (int vv = 0; vv < D; ++vv) {
        double s0 = 0.0;
        size_t idx = ((size_t)(n * H + h) * D + vv) * D + kk; /* stored [V][K] */
        if (init && init_dtype == STATE_BF16) s0 = bf2f(((const uint16_t*)init)[idx]);
        if (init && init_dtype == STATE_F32) s0 = ((const float*)init)[idx];
        S[kk * D + vv] = s0;
      }
    double a = exp((double)A_log[h]);
    for (int64_t t = cu[n]; t < cu[n + 1]; ++t) {
      size_t row = ((size_t)t * H + h) * D;
      double qn[D], kn[D], al[D], r[D];
      double sq = 0, sk = 0;
      for (int i = 0; i < D; ++i) {
        double qi = bf2f(q[row + i]), ki = bf2f(k[row + i]);
        sq += qi * qi;
        sk += ki * ki;
      }
      double rq = 1.0 / sqrt(sq + 1e-6), rk = 1.0 / sqrt(sk + 1e-6);
      for (int i = 0; i < D; ++i) {
        qn[i] = bf2f(q[row + i]) * rq;
        kn[i] = bf2f(k[row + i]) * rk;
        double x = a * ((double)bf2f(g[row + i]) + (double)dt_bias[h * D + i]);
        al[i] = exp(lower_bound / (1.0 + exp(-x)));
      }
      double b = 1.0 / (1.0 + exp(-(double)bf2f(beta[(size_t)t * H + h])));
      for (int vv = 0; vv < D; ++vv) r[vv] = bf2f(v[row + vv]);
      for (int kk = 0; kk < D; ++kk) {
        double* Sr = S + kk * D;
        double ak = al[kk], kv = kn[kk];
        for (int vv = 0; vv < D; ++vv) {
          Sr[vv] *= ak;
          r[vv] -= kv * Sr[vv];
        }
      }
      double o[D];
      for (int vv = 0; vv < D; ++vv) o[vv] = 0.0;
      for (int kk = 0; kk < D; ++kk) {
        double* Sr = S + kk * D;
        double bk = b * kn[kk], qs = qn[kk] * scale;
        for (int vv = 0; vv < D; ++vv) {
          Sr[vv] += bk * r[vv];
          o[vv] += qs * Sr[vv];
        }
      }
      for (int vv = 0; vv < D; ++vv) out_f64[row + vv] = o[vv];
    }
    if (fin_f64)
      for (int kk = 0; kk < D; ++kk)
        for (int vv = 0; vv < D; ++vv)
          fin_f64[((size_t)(n * H + h) * D + vv) * D + kk] = S[kk * D + vv];
    free(S);
  }
  return err;
}

/* ------------------------------------- chunk-16 port of tests/torch_ref.py -- */

/* tests/torch_ref.py:62-78 : sum of squares in 16 groups of 8 by FMA, xor tree */
static void l2norm_ref(const uint16_t* x, float* y /* bf16-rounded values */) {
  float part[16];
  for (int gi = 0; gi < 16; ++gi) {
    float p = 0.0f;
    for (int i = 0; i < 8; ++i) {
      float xv = bf2f(x[gi * 8 + i]);
      p = fma_via_f64(p, xv, xv);
    }
    part[gi] = p;
  }
  for (int off = 8; off >= 1; off >>= 1) {
    float nxt[16];
    for (int i = 0; i < 16; ++i) nxt[i] = part[i] + part[i ^ off];
    memcpy(part, nxt, sizeof(part));
  }
  float inv = 1.0f / sqrtf(part[0] + 1e-6f);
  for (int i = 0; i < D; ++i) y[i] = rbf(bf2f(x[i]) * inv);
}

/* tests/torch_ref.py:87-122 : (I+L)^-1 for strictly-lower fp32 L[16][16] -> bf16 values */
static void inv16_ref(const float* L, float* INV) {
  float blk[2][8][8];
  for (int b = 0; b < 2; ++b)
    for (int i = 0; i < 8; ++i)
      for (int j = 0; j < 8; ++j) blk[b][i][j] = (i == j) ? 1.0f : L[(b * 8 + i) * 16 + b * 8 + j];
  for (int b = 0; b < 2; ++b)
    for (int s = 0; s < 7; ++s) {
      float rs[8];
      for (int i = 0; i < 8; ++i) rs[i] = -blk[b][i][s];
      for (int p = 0; p < s; ++p)
        for (int i = s + 1; i < 8; ++i) blk[b][i][p] = fma_via_f64(blk[b][i][p], rs[i], blk[b][s][p]);
      for (int i = s + 1; i < 8; ++i) blk[b][i][s] = rs[i];
    }
  float P[16][16], M[16][16];
  memset(P, 0, sizeof(P));
  memset(M, 0, sizeof(M));
  for (int i = 0; i < 8; ++i)
    for (int j = 0; j < 8; ++j) {
      P[i][j] = rbf(blk[0][i][j]);
      P[8 + i][8 + j] = rbf(blk[1][i][j]);
      M[8 + i][j] = rbf(L[(8 + i) * 16 + j]);
    }
  float dc[16][16], o[16][16];
  for (int i = 0; i < 16; ++i)
    for (int j = 0; j < 16; ++j) {
      float acc = 0.0f;
      for (int l = 0; l < 16; ++l) acc += P[i][l] * M[l][j];
      dc[i][j] = acc;
    }
  for (int i = 0; i < 16; ++i)
    for (int j = 0; j < 16; ++j) {
      float acc = 0.0f;
      for (int l = 0; l < 16; ++l) acc += rbf(-dc[i][l]) * P[l][j];
      o[i][j] = acc;
    }
  for (int i = 0; i < 16; ++i)
    for (int j = 0; j < 16; ++j) INV[i * 16 + j] = rbf(P[i][j] + rbf(o[i][j]));
}

/*
 * Same tensor contract as kda_oracle_recurrence, except:
 * out_bf16 : bf16 bit patterns [T_total][H][128]
 * fin      : [N][H][128][128] bf16 or fp32 per fin_dtype, may be NULL
 * The compute state is bf16 between chunks (tests/torch_ref.py:181-183,239).
 */
int kda_oracle_chunk16(const uint16_t* q, const uint16_t* k, const uint16_t* v,
                       const uint16_t* g, const uint16_t* beta, const float* A_log,
                       const float* dt_bias, double scale, double lower_bound, const void* init,
                       int init_dtype, const int64_t* cu, int64_t N, int64_t H, int64_t seq_lo,
                       int64_t seq_hi, int64_t head_lo, int64_t head_hi, uint16_t* out_bf16,
                       void* fin, int fin_dtype, int nthreads) {
  if (!q || !k || !v || !g || !beta || !A_log || !dt_bias || !cu || !out_bf16) return -1;
  int64_t nseq = seq_hi - seq_lo, nhead = head_hi - head_lo;
  if (nseq <= 0 || nhead <= 0) return 0;
  nthreads = resolve_threads(nthreads);
  const int C = 16;
  const float scale_bf = rbf((float)scale);
  const float gate_scale = (float)(lower_bound * LOG2E);
  int err = 0;
#pragma omp parallel for num_threads(nthreads) schedule(dynamic, 1)
  for (int64_t job = 0; job < nseq * nhead; ++job) {
    int64_t n = seq_lo + job / nhead, h = head_lo + job % nhead;
    /* st[vv][kk] : bf16-valued compute state, same orientation as the API */
    float* st = (float*)malloc(sizeof(float) * D * D);
    float* buf = (float*)malloc(sizeof(float) * (10 * C * D + D * D));
    if (!st || !buf) { err = -2; free(st); free(buf); continue; }
    float *qn = buf, *kn = qn + C * D, *vc = kn + C * D, *G = vc + C * D, *kd = G + C * D,
          *qd = kd + C * D, *ki = qd + C * D, *kr = ki + C * D, *U = kr + C * D, *O = U + C * D,
          *dS = O + C * D;
    for (int i = 0; i < D * D; ++i) {
      size_t idx = (size_t)(n * H + h) * D * D + i;
      float s0 = 0.0f;
      if (init && init_dtype == STATE_BF16) s0 = bf2f(((const uint16_t*)init)[idx]);
      if (init && init_dtype == STATE_F32) s0 = rbf(((const float*)init)[idx]);
      st[i] = s0;
    }
    const float a_exp = ex2_ftz(A_log[h] * (float)LOG2E);
    int64_t bos = cu[n], eos = cu[n + 1];
    for (int64_t t0 = bos; t0 < eos; t0 += C) {
      int len = (int)((eos - t0) < C ? (eos - t0) : C);
      float bact[16], bbf[16];
      memset(buf, 0, sizeof(float) * 4 * C * D);
      for (int r = 0; r < C; ++r) {
        float blog = 0.0f;
        if (r < len) {
          size_t row = ((size_t)(t0 + r) * H + h) * D;
          l2norm_ref(q + row, qn + r * D);
          l2norm_ref(k + row, kn + r * D);
          for (int i = 0; i < D; ++i) {
            vc[r * D + i] = bf2f(v[row + i]);
            float x = bf2f(g[row + i]) + dt_bias[h * D + i];
            G[r * D + i] = gate_scale * sigmoid_tanh(a_exp * x);
          }
          blog = bf2f(beta[(size_t)(t0 + r) * H + h]);
        }
        bact[r] = sigmoid_tanh(blog);
        bbf[r] = rbf(bact[r]);
      }
      for (int r = 1; r < C; ++r)
        for (int i = 0; i < D; ++i) G[r * D + i] += G[(r - 1) * D + i];
      float gte[D], gte_bf[D];
      for (int i = 0; i < D; ++i) {
        gte[i] = ex2_ftz(G[(C - 1) * D + i]);
        gte_bf[i] = rbf(gte[i]);
      }
      for (int r = 0; r < C; ++r)
        for (int i = 0; i < D; ++i) {
          float e = rbf(ex2_ftz(G[r * D + i])), ne = rbf(ex2_ftz(-G[r * D + i]));
          kd[r * D + i] = rbf(kn[r * D + i] * e);
          qd[r * D + i] = rbf(rbf(qn[r * D + i] * e) * scale_bf);
          ki[r * D + i] = rbf(kn[r * D + i] * ne);
          kr[r * D + i] = rbf(ki[r * D + i] * gte_bf[i]);
        }
      float L[16 * 16], M[16 * 16], INV[16 * 16];
      for (int i = 0; i < C; ++i)
        for (int j = 0; j < C; ++j) {
          float al = 0.0f, am = 0.0f;
          for (int d = 0; d < D; ++d) {
            al += kd[i * D + d] * ki[j * D + d];
            am += qd[i * D + d] * ki[j * D + d];
          }
          L[i * 16 + j] = (j < i) ? al * bact[i] : 0.0f;
          M[i * 16 + j] = (j <= i) ? rbf(am) : 0.0f;
        }
      inv16_ref(L, INV);
      /* v' = bf16(bf16(v - bf16(k_decayed . S)) * bf16(beta)) ; O0 = bf16(q_decayed . S) */
      for (int r = 0; r < C; ++r)
        for (int vv = 0; vv < D; ++vv) {
          float aw = 0.0f, ao = 0.0f;
          const float* srow = st + vv * D;
          for (int d = 0; d < D; ++d) {
            aw += kd[r * D + d] * srow[d];
            ao += qd[r * D + d] * srow[d];
          }
          float vp = rbf(vc[r * D + vv] - rbf(aw));
          vc[r * D + vv] = rbf(vp * bbf[r]);
          O[r * D + vv] = rbf(ao);
        }
      for (int r = 0; r < C; ++r)
        for (int vv = 0; vv < D; ++vv) {
          float acc = 0.0f;
          for (int j = 0; j < C; ++j) acc += INV[r * 16 + j] * vc[j * D + vv];
          U[r * D + vv] = rbf(acc);
        }
      for (int r = 0; r < len; ++r) {
        size_t row = ((size_t)(t0 + r) * H + h) * D;
        for (int vv = 0; vv < D; ++vv) {
          float acc = 0.0f;
          for (int j = 0; j < C; ++j) acc += M[r * 16 + j] * U[j * D + vv];
          out_bf16[row + vv] = f2bf(O[r * D + vv] + rbf(acc));
        }
      }
      for (int d = 0; d < D; ++d)
        for (int vv = 0; vv < D; ++vv) {
          float acc = 0.0f;
          for (int j = 0; j < C; ++j) acc += kr[j * D + d] * U[j * D + vv];
          dS[vv * D + d] = acc;
        }
      for (int vv = 0; vv < D; ++vv)
        for (int d = 0; d < D; ++d)
          st[vv * D + d] = rbf(fma_via_f64(dS[vv * D + d], st[vv * D + d], gte[d]));
    }
    if (fin)
      for (int i = 0; i < D * D; ++i) {
        size_t idx = (size_t)(n * H + h) * D * D + i;
        if (fin_dtype == STATE_BF16) ((uint16_t*)fin)[idx] = f2bf(st[i]);
        if (fin_dtype == STATE_F32) ((float*)fin)[idx] = st[i];
      }
    free(st);
    free(buf);
  }
  return err;
}

/* ------------------------- fp64 operands of the chunk-C WY formulation ------ */

/*
 * For one head h and one chunk of `len` (<= C <= 64) tokens starting at token t0:
 *   Gc[i]   = sum_{j<=i} log-decay of token j          (natural log, per channel)
 *   kpp[i]  = khat_i * exp(Gc[i])            [C][128]   keys decayed from the chunk start
 *   qpp[i]  = qhat_i * exp(Gc[i]) * scale    [C][128]
 *   kr[i]   = khat_i * exp(Gc[last]-Gc[i])   [C][128]   keys decayed to the chunk end
 *   ec      = exp(Gc[last])                  [128]      whole-chunk decay
 *   A       = tril(k k^T with decay exp(Gc[i]-Gc[j]), -1) * beta_i ; T = (I+A)^-1
 *   wp      = T diag(beta) kpp               [C][128]
 *   up      = T diag(beta) v                 [C][128]
 *   mqk     = tril(q k^T with decay, 0)*scale [C][C]
 * so that, with S the state at the chunk start ([K][V]):
 *   U = up - wp S ;  out = qpp S + mqk U ;  S' = diag(ec) S + kr^T U.
 * Rows >= len are zero.  Chunk decomposition restates tests/torch_ref.py:196-241
 * algebraically (U = INV (v - k_decayed S) beta  ==  up - wp S).
 */
int kda_oracle_chunk_operands(const uint16_t* q, const uint16_t* k, const uint16_t* v,
                              const uint16_t* g, const uint16_t* beta, const float* A_log,
                              const float* dt_bias, double scale, double lower_bound, int64_t H,
                              int64_t h, int64_t t0, int len, int C, double* kpp, double* qpp,
                              double* kr, double* ec, double* wp, double* up, double* mqk) {
  if (C > 64 || len > C || len < 0) return -1;
  static const int MAXC = 64;
  double(*Gc)[D] = malloc(sizeof(double) * MAXC * D);
  double(*kn)[D] = malloc(sizeof(double) * MAXC * D);
  double(*qn)[D] = malloc(sizeof(double) * MAXC * D);
  double A[64][64], T[64][64], b[64];
  if (!Gc || !kn || !qn) return -2;
  memset(Gc, 0, sizeof(double) * MAXC * D);
  memset(kn, 0, sizeof(double) * MAXC * D);
  memset(qn, 0, sizeof(double) * MAXC * D);
  double a = exp((double)A_log[h]);
  for (int r = 0; r < C; ++r) {
    b[r] = 0.5;
    if (r < len) {
      size_t row = ((size_t)(t0 + r) * H + h) * D;
      double sq = 0, sk = 0;
      for (int i = 0; i < D; ++i) {
        double qi = bf2f(q[row + i]), ki = bf2f(k[row + i]);
        sq += qi * qi;
        sk += ki * ki;
      }
      double rq = 1.0 / sqrt(sq + 1e-6), rk = 1.0 / sqrt(sk + 1e-6);
      for (int i = 0; i < D; ++i) {
        qn[r][i] = bf2f(q[row + i]) * rq;
        kn[r][i] = bf2f(k[row + i]) * rk;
        double x = a * ((double)bf2f(g[row + i]) + (double)dt_bias[h * D + i]);
        Gc[r][i] = lower_bound / (1.0 + exp(-x));
      }
      b[r] = 1.0 / (1.0 + exp(-(double)bf2f(beta[(size_t)(t0 + r) * H + h])));
    }
    if (r > 0)
      for (int i = 0; i < D; ++i) Gc[r][i] += Gc[r - 1][i];
  }
  for (int i = 0; i < D; ++i) ec[i] = exp(Gc[C - 1][i]);
  for (int r = 0; r < C; ++r)
    for (int i = 0; i < D; ++i) {
      kpp[r * D + i] = kn[r][i] * exp(Gc[r][i]);
      qpp[r * D + i] = qn[r][i] * exp(Gc[r][i]) * scale;
      kr[r * D + i] = kn[r][i] * exp(Gc[C - 1][i] - Gc[r][i]);
    }
  for (int i = 0; i < C; ++i)
    for (int j = 0; j < C; ++j) {
      double sa = 0, sm = 0;
      if (j <= i)
        for (int d = 0; d < D; ++d) {
          double e = exp(Gc[i][d] - Gc[j][d]);
          sa += kn[i][d] * kn[j][d] * e;
          sm += qn[i][d] * kn[j][d] * e;
        }
      A[i][j] = (j < i) ? sa * b[i] : 0.0;
      mqk[i * C + j] = (j <= i) ? sm * scale : 0.0;
    }
  for (int c = 0; c < C; ++c)
    for (int i = 0; i < C; ++i) {
      double acc = (i == c) ? 1.0 : 0.0;
      for (int j = 0; j < i; ++j) acc -= A[i][j] * T[j][c];
      T[i][c] = acc;
    }
  for (int i = 0; i < C; ++i)
    for (int d = 0; d < D; ++d) {
      double sw = 0, su = 0;
      for (int j = 0; j <= i; ++j) {
        double tb = T[i][j] * b[j];
        sw += tb * kpp[j * D + d];
        double vv = 0.0;
        if (j < len) vv = bf2f(v[((size_t)(t0 + j) * H + h) * D + d]);
        su += tb * vv;
      }
      wp[i * D + d] = sw;
      up[i * D + d] = su;
    }
  free(Gc);
  free(kn);
  free(qn);
  return 0;
}
