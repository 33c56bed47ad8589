// CPU oracle for the LLM-step kernels of tessel (kernels/llm.tl, plus `matmul`
// of kernels/matmul.tl and `flash_attention` / `paged_attention` of
// kernels/attention.tl), restated op by op under the semantics of tessel's IR
// interpreter (src/interp.rs).
//
// THIS IS TEST INFRASTRUCTURE, NOT PRODUCT CODE. Only the test-suite, the
// smoke check and the CPU-baseline leg of the benchmark may load it; the
// shipped library never does.
//
// Pin status. The reference stores no golden vectors for these kernels (every
// expectation in its tests is recomputed from seeded inputs) and its Rust
// sources cannot be built where this oracle was written, so bit-level parity
// of the kernel restatements is UNPINNED ("parity unpinned"). What is pinned:
//   * f16 rounding against the known-answer values of src/half.rs:69-77 and,
//     exhaustively, against kf2h/kh2f of src/prelude.cuh:104-140 compiled
//     from the reference tree (oracle/_ref);
//   * every kernel against the plain f64 procedures the reference's own tests
//     use (tests/common/mod.rs:45-173), on the same seeded xorshift inputs
//     (src/bench.rs:13-35) and at the reference's tolerances
//     (tests/interp.rs:63-136, examples/metal_cases.rs:159-324).
//
// Interpreter rules followed throughout (src/interp.rs:46-59, :84-87): every
// value is rounded to its dtype after every op; `sum` and `dot` add in f64 and
// round once to f32 (src/interp.rs:251-295); exp/sqrt are evaluated in f32
// (src/interp.rs:171-181); loads outside an array read 0, stores outside are
// dropped (src/interp.rs:93-117, :297-314). An f64 product/sum/quotient of two
// f32 values rounded to f32 equals the f32 operation (53 >= 2*24+2), so plain
// f32 arithmetic is used where the interpreter computes in f64 and rounds.
//
// Build: g++ -O2 -pthread -ffp-contract=off -shared -fPIC (see oracle/Makefile).
// -ffp-contract=off matters: a fused multiply-add would skip a rounding the
// interpreter performs.

#include <algorithm>
#include <atomic>
#include <cmath>
#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <limits>
#include <thread>
#include <vector>

namespace {

typedef uint16_t h16;

// Threads used by par_for: ORACLE_THREADS, else the hardware's count.
int n_threads() {
  static int n = [] {
    const char* e = std::getenv("ORACLE_THREADS");
    int v = e ? std::atoi(e) : (int)std::thread::hardware_concurrency();
    return v > 0 ? v : 1;
  }();
  return n;
}

// Runs fn(i) for i in [0, n) on n_threads() threads, items handed out in
// chunks from a shared counter. Every item writes its own outputs only.
template <class F>
void par_for(long long n, F fn) {
  const int nt = (int)std::min<long long>(n_threads(), n);
  if (nt <= 1) {
    for (long long i = 0; i < n; ++i) fn(i);
    return;
  }
  std::atomic<long long> next(0);
  const long long chunk = std::max<long long>(1, n / (nt * 8));
  auto work = [&]() {
    for (;;) {
      const long long b = next.fetch_add(chunk);
      if (b >= n) return;
      const long long e = std::min(n, b + chunk);
      for (long long i = b; i < e; ++i) fn(i);
    }
  };
  std::vector<std::thread> ts;
  for (int t = 1; t < nt; ++t) ts.emplace_back(work);
  work();
  for (auto& t : ts) t.join();
}

// IEEE binary16 <-> binary32, round to nearest even, following the cases of
// src/half.rs:3-63 (NaN keeps a quiet bit, overflow gives infinity,
// subnormals are produced and consumed).
inline h16 f2h(float f) {
  uint32_t x;
  std::memcpy(&x, &f, 4);
  const uint32_t sign = (x >> 16) & 0x8000u;
  const uint32_t e = (x >> 23) & 0xffu;
  uint32_t man = x & 0x7fffffu;
  if (e == 0xffu) return (h16)(sign | 0x7c00u | (man ? 0x200u : 0u));
  const int exp = (int)e - 127 + 15;
  if (exp >= 31) return (h16)(sign | 0x7c00u);
  if (exp <= 0) {
    if (exp < -10) return (h16)sign;
    man |= 0x800000u;
    const uint32_t shift = (uint32_t)(14 - exp);
    uint32_t h = man >> shift;
    const uint32_t rem = man & ((1u << shift) - 1u);
    const uint32_t half = 1u << (shift - 1);
    if (rem > half || (rem == half && (h & 1u))) h += 1;
    return (h16)(sign | h);
  }
  uint32_t h = ((uint32_t)exp << 10) | (man >> 13);
  const uint32_t rem = man & 0x1fffu;
  if (rem > 0x1000u || (rem == 0x1000u && (h & 1u))) h += 1;  // may carry into the exponent: correct
  return (h16)(sign | h);
}

inline float h2f(h16 h) {
  const uint32_t sign = ((uint32_t)h & 0x8000u) << 16;
  const uint32_t exp = (h >> 10) & 0x1fu;
  uint32_t man = h & 0x3ffu;
  uint32_t x;
  if (exp == 0) {
    if (man == 0) {
      x = sign;
    } else {
      int e = 1;
      while (!(man & 0x400u)) {
        man <<= 1;
        e -= 1;
      }
      x = sign | ((uint32_t)(e + 127 - 15) << 23) | ((man & 0x3ffu) << 13);
    }
  } else if (exp == 31) {
    x = sign | 0x7f800000u | (man << 13);
  } else {
    x = sign | ((exp + 127 - 15) << 23) | (man << 13);
  }
  float f;
  std::memcpy(&f, &x, 4);
  return f;
}

inline float r16(float x) { return h2f(f2h(x)); }

const float NEG_INF = -std::numeric_limits<float>::infinity();

// max as src/interp.rs:207-213 defines it: keeps x when y is NaN.
inline float imax(float x, float y) { return (x >= y || y != y) ? x : y; }

// The rotation of kernels/llm.tl:85-88 / :102-105 on one pair, every product
// and the sum rounded on its own.
inline void rotate(float x1, float x2, float c, float s, h16* y1, h16* y2) {
  const float a = x1 * c, b = x2 * s;
  const float d = x2 * c, e = x1 * s;
  *y1 = f2h(a - b);
  *y2 = f2h(d + e);
}

// One row of kernels/llm.tl:19-25 (and :175-182): x -> f16(x * rsqrt(ms+eps) * w).
void norm_row(const float* x, const h16* w, h16* y, float eps, int dm) {
  double ss = 0.0;
  for (int c = 0; c < dm; ++c) ss += (double)(x[c] * x[c]);
  const float sum = (float)ss;
  const float ms = sum / (float)dm;
  const float r = 1.0f / std::sqrt(ms + eps);  // src/interp.rs:176
  for (int c = 0; c < dm; ++c) y[c] = f2h((x[c] * r) * h2f(w[c]));
}

// acc[n] (+)= x[k..k+bk) . w[n][k..k+bk), one f64 sum per BK block rounded to
// f32 (src/interp.rs:280-295 applied to kernels/llm.tl:33-35).
inline float dot_blocks(const float* x, const float* w, int K, int bk) {
  float acc = 0.0f;
  for (int k0 = 0; k0 < K; k0 += bk) {
    const int k1 = k0 + bk < K ? k0 + bk : K;
    double s = 0.0;
    for (int k = k0; k < k1; ++k) s += (double)x[k] * (double)w[k];
    acc = (float)((double)acc + s);
  }
  return acc;
}

std::vector<float> widen(const h16* p, size_t n) {
  std::vector<float> v(n);
  const long long rows = (long long)((n + 4095) / 4096);
  par_for(rows, [&](long long r) {
    const size_t e = std::min(n, (size_t)(r + 1) * 4096);
    for (size_t i = (size_t)r * 4096; i < e; ++i) v[i] = h2f(p[i]);
  });
  return v;
}

}  // namespace

extern "C" {

// ---- f16 -------------------------------------------------------------------
uint16_t orc_f2h(float f) { return f2h(f); }
float orc_h2f(uint16_t h) { return h2f(h); }
void orc_f2h_n(const float* x, uint16_t* y, long long n) {
  for (long long i = 0; i < n; ++i) y[i] = f2h(x[i]);
}
void orc_h2f_n(const uint16_t* x, float* y, long long n) {
  for (long long i = 0; i < n; ++i) y[i] = h2f(x[i]);
}

// ---- kernels/llm.tl:10-16 ----------------------------------------------------
void orc_embed(const int32_t* tok, const uint16_t* E, float* X, int T, int V, int Dm) {
  for (int t = 0; t < T; ++t) {
    const int row = tok[t];
    for (int c = 0; c < Dm; ++c) X[(size_t)t * Dm + c] = (row >= 0 && row < V) ? h2f(E[(size_t)row * Dm + c]) : 0.0f;
  }
}

// ---- kernels/llm.tl:19-25 ----------------------------------------------------
void orc_rmsnorm(const float* X, const uint16_t* W, uint16_t* Y, float eps, int T, int Dm) {
  par_for(T, [&](long long t) { norm_row(X + (size_t)t * Dm, W, Y + (size_t)t * Dm, eps, Dm); });
}

// ---- kernels/llm.tl:175-182 --------------------------------------------------
void orc_rmsnorm_rows(const float* X, const int32_t* idx, const uint16_t* W, uint16_t* Y, float eps, int T, int B,
                      int Dm) {
  std::vector<float> zero(Dm, 0.0f);
  for (int b = 0; b < B; ++b) {
    const int r = idx[b];
    norm_row((r >= 0 && r < T) ? X + (size_t)r * Dm : zero.data(), W, Y + (size_t)b * Dm, eps, Dm);
  }
}

// ---- kernels/llm.tl:28-58: linear / linear_residual / logits -----------------
// mode 0: Y f16 = acc; mode 1: R f32 += acc; mode 2: Y f32 = acc.
void orc_linear_family(const uint16_t* X, const uint16_t* W, void* out, int M, int N, int K, int bk, int mode) {
  std::vector<float> xf = widen(X, (size_t)M * K), wf = widen(W, (size_t)N * K);
  par_for((long long)M * N, [&](long long o) {
    const long long i = o / N, j = o % N;
    const float acc = dot_blocks(&xf[(size_t)i * K], &wf[(size_t)j * K], K, bk);
    if (mode == 0)
      ((uint16_t*)out)[o] = f2h(acc);
    else if (mode == 1)
      ((float*)out)[o] = ((float*)out)[o] + acc;
    else
      ((float*)out)[o] = acc;
  });
}

// ---- kernels/llm.tl:62-73 ----------------------------------------------------
void orc_gate_up(const uint16_t* X, const uint16_t* Wg, const uint16_t* Wu, uint16_t* Y, int M, int F, int K, int bk) {
  std::vector<float> xf = widen(X, (size_t)M * K), gf = widen(Wg, (size_t)F * K), uf = widen(Wu, (size_t)F * K);
  par_for((long long)M * F, [&](long long o) {
    const long long i = o / F, j = o % F;
    const float g = dot_blocks(&xf[(size_t)i * K], &gf[(size_t)j * K], K, bk);
    const float u = dot_blocks(&xf[(size_t)i * K], &uf[(size_t)j * K], K, bk);
    const float e = std::exp(-g);
    const float d = 1.0f + e;
    const float q = g / d;
    Y[o] = f2h(q * u);
  });
}

// ---- kernels/matmul.tl:3-17: C f16 = A[M,K] B[K,N], both row-major ------------
void orc_matmul(const uint16_t* A, const uint16_t* B, uint16_t* C, int M, int N, int K, int bk) {
  std::vector<float> af = widen(A, (size_t)M * K);
  std::vector<float> bt((size_t)N * K);
  par_for(N, [&](long long j) {
    for (int k = 0; k < K; ++k) bt[(size_t)j * K + k] = h2f(B[(size_t)k * N + j]);
  });
  par_for((long long)M * N, [&](long long o) {
    const long long i = o / N, j = o % N;
    C[o] = f2h(dot_blocks(&af[(size_t)i * K], &bt[(size_t)j * K], K, bk));
  });
}

// Rows [r0, r1) x columns [c0, c1) of orc_matmul, for timing a bounded sample
// of a large product. Cs is the [r1-r0, c1-c0] result.
void orc_matmul_block(const uint16_t* A, const uint16_t* B, uint16_t* Cs, int M, int N, int K, int bk, int r0, int r1,
                      int c0, int c1) {
  (void)M;
  const int nr = r1 - r0, nc = c1 - c0;
  std::vector<float> af = widen(A + (size_t)r0 * K, (size_t)nr * K);
  std::vector<float> bt((size_t)nc * K);
  par_for(nc, [&](long long j) {
    for (int k = 0; k < K; ++k) bt[(size_t)j * K + k] = h2f(B[(size_t)k * N + c0 + j]);
  });
  par_for((long long)nr * nc, [&](long long o) {
    const long long i = o / nc, j = o % nc;
    Cs[o] = f2h(dot_blocks(&af[(size_t)i * K], &bt[(size_t)j * K], K, bk));
  });
}

// ---- kernels/llm.tl:78-88 ----------------------------------------------------
void orc_rope_q(const uint16_t* QKV, const int32_t* pos, const float* C, const float* S, uint16_t* Q, int T, int W,
                int NPOS, int H, int D) {
  const int d2 = D / 2;
  for (int t = 0; t < T; ++t) {
    const int p = pos[t];
    const bool in = p >= 0 && p < NPOS;
    for (int h = 0; h < H; ++h)
      for (int i = 0; i < d2; ++i) {
        const float c = in ? C[(size_t)p * d2 + i] : 0.0f, s = in ? S[(size_t)p * d2 + i] : 0.0f;
        const int a = h * D + i, b = h * D + d2 + i;
        const float x1 = a < W ? h2f(QKV[(size_t)t * W + a]) : 0.0f;
        const float x2 = b < W ? h2f(QKV[(size_t)t * W + b]) : 0.0f;
        rotate(x1, x2, c, s, &Q[((size_t)t * H + h) * D + i], &Q[((size_t)t * H + h) * D + d2 + i]);
      }
  }
}

// ---- kernels/llm.tl:93-112 ---------------------------------------------------
void orc_kv_write(const uint16_t* QKV, const int32_t* pos, const int32_t* slot, const float* C, const float* S,
                  uint16_t* Kc, uint16_t* Vc, uint16_t* Kd, uint16_t* Vd, int T, int W, int NPOS, int NS, int G,
                  int D) {
  const int d2 = D / 2;
  for (int t = 0; t < T; ++t) {
    const int p = pos[t], at = slot[t];
    const bool in = p >= 0 && p < NPOS, keep = at >= 0 && at < NS;
    for (int g = 0; g < G; ++g) {
      const int k0 = W - 2 * G * D + g * D;
      for (int i = 0; i < d2; ++i) {
        const float c = in ? C[(size_t)p * d2 + i] : 0.0f, s = in ? S[(size_t)p * d2 + i] : 0.0f;
        const float x1 = h2f(QKV[(size_t)t * W + k0 + i]), x2 = h2f(QKV[(size_t)t * W + k0 + d2 + i]);
        h16 y1, y2;
        rotate(x1, x2, c, s, &y1, &y2);
        Kd[((size_t)t * G + g) * D + i] = y1;
        Kd[((size_t)t * G + g) * D + d2 + i] = y2;
        if (keep) {
          Kc[((size_t)at * G + g) * D + i] = y1;
          Kc[((size_t)at * G + g) * D + d2 + i] = y2;
        }
      }
      for (int i = 0; i < D; ++i) {
        const h16 v = QKV[(size_t)t * W + k0 + G * D + i];
        Vd[((size_t)t * G + g) * D + i] = v;
        if (keep) Vc[((size_t)at * G + g) * D + i] = v;
      }
    }
  }
}

// ---- kernels/llm.tl:150-172 (and kernels/attention.tl:29-51 with G == H) ------
void orc_decode_attention(const uint16_t* Q, const uint16_t* Kc, const uint16_t* Vc, const int32_t* table,
                          const int32_t* lens, uint16_t* O, float scale, int B, int H, int G, int D, int NP, int P,
                          int MP) {
  par_for((long long)B * H, [&](long long bh) {
      const int b = (int)(bh / H), h = (int)(bh % H);
      const int g = h / (H / G), n = lens[b];
      std::vector<float> q(D), acc(D, 0.0f), sc(P), p(P);
      for (int d = 0; d < D; ++d) q[d] = h2f(Q[((size_t)b * H + h) * D + d]);
      float m = NEG_INF, l = 0.0f;
      for (int t = 0; t < n; t += P) {
        const int col = t / P;
        const int page = (col >= 0 && col < MP) ? table[(size_t)b * MP + col] : 0;
        const bool in = page >= 0 && page < NP;
        float blockmax = NEG_INF;
        for (int i = 0; i < P; ++i) {
          double s = 0.0;
          if (in)
            for (int d = 0; d < D; ++d) s += (double)(h2f(Kc[(((size_t)page * P + i) * G + g) * D + d]) * q[d]);
          const float v = (float)s * scale;
          sc[i] = (t + i < n) ? v : NEG_INF;
          blockmax = imax(blockmax, sc[i]);  // f64 max fold of src/interp.rs:266
        }
        const float m2 = imax(m, blockmax);
        double ps = 0.0;
        for (int i = 0; i < P; ++i) {
          p[i] = std::exp(sc[i] - m2);
          ps += (double)p[i];
        }
        const float a = std::exp(m - m2);
        l = l * a + (float)ps;
        for (int d = 0; d < D; ++d) {
          double s = 0.0;
          if (in)
            for (int i = 0; i < P; ++i) s += (double)(p[i] * h2f(Vc[(((size_t)page * P + i) * G + g) * D + d]));
          acc[d] = acc[d] * a + (float)s;
        }
        m = m2;
      }
      for (int d = 0; d < D; ++d) O[((size_t)b * H + h) * D + d] = f2h(acc[d] / l);
  });
}

// ---- kernels/llm.tl:116-145; `plain` selects kernels/attention.tl:4-24 ---------
// Packed layout: Q,O [S,H,D], K,V [S,G,D]. Plain layout ([H,S,D], no starts,
// running maximum from -inf) is expressed through the strides below.
static void attention_rows(const uint16_t* Q, const uint16_t* K, const uint16_t* V, const int32_t* starts, uint16_t* O,
                           float scale, int S, int H, int G, int D, int BM, int BN, bool plain, int only_h0,
                           int only_h1, int only_blk0, int only_blk1) {
  const size_t qs = plain ? (size_t)D : (size_t)H * D;        // row stride of Q/O
  const size_t qh = plain ? (size_t)S * D : (size_t)D;        // head stride of Q/O
  const size_t ks = plain ? (size_t)D : (size_t)G * D;        // row stride of K/V
  const size_t kh = plain ? (size_t)S * D : (size_t)D;        // head stride of K/V
  const int nblk = (S + BM - 1) / BM;
  const int b0 = only_blk0 < 0 ? 0 : only_blk0, b1 = only_blk1 < 0 ? nblk : only_blk1;
  const int nb = b1 - b0;
  par_for((long long)(only_h1 - only_h0) * nb, [&](long long it) {
      const int h = only_h0 + (int)(it / nb), blk = b0 + (int)(it % nb);
      const int i0 = blk * BM;
      const int g = plain ? h : h / (H / G);
      std::vector<float> q((size_t)BM * D), acc((size_t)BM * D, 0.0f), m(BM), l(BM, 0.0f), s(BN), p16(BN);
      std::vector<int> st(BM);
      for (int r = 0; r < BM; ++r) {
        const int row = i0 + r;
        for (int d = 0; d < D; ++d) q[(size_t)r * D + d] = row < S ? h2f(Q[row * qs + h * qh + d]) : 0.0f;
        st[r] = (plain || row >= S) ? 0 : starts[row];
        m[r] = plain ? NEG_INF : -1e30f;
      }
      const int lo = plain ? 0 : starts[i0];
      const int hi = i0 + BM < S ? i0 + BM : S;
      std::vector<float> kb((size_t)BN * D), vb((size_t)BN * D);
      for (int j = lo; j < hi; j += BN) {
        for (int c = 0; c < BN; ++c) {
          const int col = j + c;
          const bool in = col >= 0 && col < S;
          for (int d = 0; d < D; ++d) {
            kb[(size_t)c * D + d] = in ? h2f(K[col * ks + g * kh + d]) : 0.0f;
            vb[(size_t)c * D + d] = in ? h2f(V[col * ks + g * kh + d]) : 0.0f;
          }
        }
        for (int r = 0; r < BM; ++r) {
          const int row = i0 + r;
          float bm = NEG_INF;
          for (int c = 0; c < BN; ++c) {
            const int col = j + c;
            double d0 = 0.0;
            for (int d = 0; d < D; ++d) d0 += (double)q[(size_t)r * D + d] * (double)kb[(size_t)c * D + d];
            const float v = (float)d0 * scale;
            const bool ok = col <= row && col >= st[r] && col < S;
            s[c] = ok ? v : NEG_INF;
            bm = imax(bm, s[c]);
          }
          const float m2 = imax(m[r], bm);
          double ps = 0.0;
          for (int c = 0; c < BN; ++c) {
            const float e = std::exp(s[c] - m2);
            ps += (double)e;
            p16[c] = r16(e);  // f16(p) of kernels/llm.tl:143
          }
          const float a = std::exp(m[r] - m2);
          l[r] = l[r] * a + (float)ps;
          for (int d = 0; d < D; ++d) {
            double pv = 0.0;
            for (int c = 0; c < BN; ++c) pv += (double)p16[c] * (double)vb[(size_t)c * D + d];
            acc[(size_t)r * D + d] = acc[(size_t)r * D + d] * a + (float)pv;
          }
          m[r] = m2;
        }
      }
      for (int r = 0; r < BM; ++r) {
        const int row = i0 + r;
        if (row >= S) continue;
        for (int d = 0; d < D; ++d) O[row * qs + h * qh + d] = f2h(acc[(size_t)r * D + d] / l[r]);
      }
  });
}

void orc_prefill_attention(const uint16_t* Q, const uint16_t* K, const uint16_t* V, const int32_t* starts, uint16_t* O,
                           float scale, int S, int H, int G, int D, int BM, int BN) {
  attention_rows(Q, K, V, starts, O, scale, S, H, G, D, BM, BN, false, 0, H, -1, -1);
}

void orc_flash_attention(const uint16_t* Q, const uint16_t* K, const uint16_t* V, uint16_t* O, float scale, int H,
                         int S, int D, int BM, int BN) {
  attention_rows(Q, K, V, nullptr, O, scale, S, H, H, D, BM, BN, true, 0, H, -1, -1);
}

// Heads [h0,h1) and query blocks [blk0,blk1) only: a bounded sample for timing.
void orc_flash_attention_part(const uint16_t* Q, const uint16_t* K, const uint16_t* V, uint16_t* O, float scale, int H,
                              int S, int D, int BM, int BN, int h0, int h1, int blk0, int blk1) {
  attention_rows(Q, K, V, nullptr, O, scale, S, H, H, D, BM, BN, true, h0, h1, blk0, blk1);
}

// ---- src/llm/mod.rs:116-129 ---------------------------------------------------
void orc_rope_tables(float* C, float* S, int max_pos, int head_dim, float theta) {
  const int h = head_dim / 2;
  for (int p = 0; p < max_pos; ++p)
    for (int i = 0; i < h; ++i) {
      const double inv = std::pow((double)theta, -((double)(2 * i)) / (double)head_dim);
      const double a = (double)p * inv;
      C[(size_t)p * h + i] = (float)std::cos(a);
      S[(size_t)p * h + i] = (float)std::sin(a);
    }
}

// ---- src/llm/mod.rs:132-140: first maximum wins --------------------------------
int orc_argmax(const float* x, int n) {
  int best = 0;
  for (int i = 0; i < n; ++i)
    if (x[i] > x[best]) best = i;
  return best;
}

// ---- src/llm/reference.rs:38-108: the f32 model, one sequence ------------------
// Weights are f16 bits laid out as src/llm/mod.rs:55-78 describes. `layers`
// points at 7 arrays per layer: attn_norm, wqkv, wo, mlp_norm, wg, wu, wd.
// logits_out is [ntok, vocab].
void orc_reference_forward(const uint16_t* embed, const uint16_t* const* layers, const uint16_t* norm,
                           const uint16_t* head, const int32_t* tokens, int ntok, float* logits_out, int dim,
                           int nlayers, int nh, int ng, int hd, int ffn, int vocab, float eps, float theta,
                           int max_pos) {
  const int qkvw = (nh + 2 * ng) * hd, half = hd / 2;
  std::vector<float> C((size_t)max_pos * half), S((size_t)max_pos * half);
  orc_rope_tables(C.data(), S.data(), max_pos, hd, theta);
  struct L {
    std::vector<float> n1, wqkv, wo, n2, wg, wu, wd;
  };
  std::vector<L> ls(nlayers);
  for (int i = 0; i < nlayers; ++i) {
    const uint16_t* const* p = layers + 7 * i;
    ls[i].n1 = widen(p[0], dim);
    ls[i].wqkv = widen(p[1], (size_t)qkvw * dim);
    ls[i].wo = widen(p[2], (size_t)dim * nh * hd);
    ls[i].n2 = widen(p[3], dim);
    ls[i].wg = widen(p[4], (size_t)ffn * dim);
    ls[i].wu = widen(p[5], (size_t)ffn * dim);
    ls[i].wd = widen(p[6], (size_t)dim * ffn);
  }
  std::vector<float> nf = widen(norm, dim), hf = widen(head, (size_t)vocab * dim);
  auto matvec = [](const std::vector<float>& w, const std::vector<float>& x, int rows) {
    const int cols = (int)x.size();
    std::vector<float> y(rows);
    par_for(rows, [&](long long r) {
      float s = 0.0f;  // f32 running sum, as Iterator::sum::<f32>() does
      for (int c = 0; c < cols; ++c) s += w[(size_t)r * cols + c] * x[c];
      y[r] = s;
    });
    return y;
  };
  auto rms = [&](const std::vector<float>& x, const std::vector<float>& w) {
    float ss = 0.0f;
    for (float v : x) ss += v * v;
    const float sc = 1.0f / std::sqrt(ss / (float)x.size() + eps);
    std::vector<float> y(x.size());
    for (size_t i = 0; i < x.size(); ++i) y[i] = x[i] * sc * w[i];
    return y;
  };
  auto rope = [&](float* x, int nheads, int pos) {
    for (int h = 0; h < nheads; ++h)
      for (int i = 0; i < half; ++i) {
        const float cs = C[(size_t)pos * half + i], sn = S[(size_t)pos * half + i];
        const float a = x[h * hd + i], b = x[h * hd + i + half];
        x[h * hd + i] = a * cs - b * sn;
        x[h * hd + i + half] = b * cs + a * sn;
      }
  };
  std::vector<std::vector<std::vector<float>>> kc(nlayers), vc(nlayers);
  const float rs = std::sqrt((float)hd);
  for (int pos = 0; pos < ntok; ++pos) {
    const int t = tokens[pos];
    std::vector<float> x(dim);
    for (int c = 0; c < dim; ++c) x[c] = h2f(embed[(size_t)t * dim + c]);
    for (int li = 0; li < nlayers; ++li) {
      L& w = ls[li];
      std::vector<float> h = rms(x, w.n1);
      std::vector<float> qkv = matvec(w.wqkv, h, qkvw);
      std::vector<float> q(qkv.begin(), qkv.begin() + nh * hd);
      std::vector<float> k(qkv.begin() + nh * hd, qkv.begin() + (nh + ng) * hd);
      std::vector<float> v(qkv.begin() + (nh + ng) * hd, qkv.end());
      rope(q.data(), nh, pos);
      rope(k.data(), ng, pos);
      kc[li].push_back(k);
      vc[li].push_back(v);
      std::vector<float> o((size_t)nh * hd, 0.0f);
      for (int hh = 0; hh < nh; ++hh) {
        const int g = hh / (nh / ng);
        const int n = (int)kc[li].size();
        std::vector<float> sc(n);
        float mx = NEG_INF;
        for (int j = 0; j < n; ++j) {
          float s = 0.0f;
          for (int d = 0; d < hd; ++d) s += kc[li][j][g * hd + d] * q[hh * hd + d];
          sc[j] = s / rs;
          mx = std::fmax(mx, sc[j]);
        }
        float z = 0.0f;
        for (int j = 0; j < n; ++j) {
          sc[j] = std::exp(sc[j] - mx);
          z += sc[j];
        }
        for (int j = 0; j < n; ++j)
          for (int d = 0; d < hd; ++d) o[hh * hd + d] += sc[j] / z * vc[li][j][g * hd + d];
      }
      std::vector<float> po = matvec(w.wo, o, dim);
      for (int c = 0; c < dim; ++c) x[c] += po[c];
      h = rms(x, w.n2);
      std::vector<float> gg = matvec(w.wg, h, ffn), uu = matvec(w.wu, h, ffn), a(ffn);
      for (int i = 0; i < ffn; ++i) a[i] = gg[i] / (1.0f + std::exp(-gg[i])) * uu[i];
      std::vector<float> pd = matvec(w.wd, a, dim);
      for (int c = 0; c < dim; ++c) x[c] += pd[c];
    }
    std::vector<float> lg = matvec(hf, rms(x, nf), vocab);
    std::memcpy(logits_out + (size_t)pos * vocab, lg.data(), (size_t)vocab * 4);
  }
}

// ---- src/bench.rs:13-35: the seeded generator every reference test uses --------
uint64_t orc_rng_seed(uint64_t seed) { return (seed * 0x9e3779b97f4a7c15ull) | 1ull; }

// Draws n uniforms in [-1, 1) and advances *state (xorshift 13/7/17, top 24 bits).
void orc_rng_uniform(uint64_t* state, float* out, long long n) {
  uint64_t s = *state;
  for (long long i = 0; i < n; ++i) {
    s ^= s << 13;
    s ^= s >> 7;
    s ^= s << 17;
    out[i] = ((float)(s >> 40) / (float)(1ull << 24)) * 2.0f - 1.0f;
  }
  *state = s;
}

int orc_threads(void) { return n_threads(); }

}  // extern "C"
