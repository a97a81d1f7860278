/* TEST INFRASTRUCTURE -- PARITY UNPINNED.
 *
 * A second, independent CPU restatement of rai's decoder forward pass in plain C (float32, IEEE
 * arithmetic, no fast-math), written from the reference's sources and not from oracle/rai_cpu.py:
 * the two are checked against each other in tests/test_oracle.py, so that a misreading of the
 * reference would have to be made twice, in two languages, to go unnoticed.  Like everything under
 * oracle/ it may be used by tests/, __graft_entry__.smoke() and bench.py's CPU baseline only.
 *
 * The reference cannot be built here (Rust, no toolchain) and holds no golden vectors for this
 * path, so neither restatement is pinned to outputs of the reference itself.
 *
 * What is restated, op for op, in the reference's order:
 *   Model::fwd           rai-models/src/llm/qwen2.rs:338-359, gemma.rs:364-386, phi3.rs:308-323, phi2.rs:334-347
 *   DecoderLayer::fwd    qwen2.rs:255-266, gemma.rs:292-303, phi3.rs:243-251, phi2.rs:293-299 (parallel block)
 *   Attention::fwd       qwen2.rs:170-221, gemma.rs:203-254, phi3.rs:163-211, phi2.rs:202-264
 *   RotaryEmbedding      qwen2.rs:40-72, gemma.rs:71-103, phi3.rs:40-75, phi2.rs:44-78
 *   MLP                  qwen2.rs:100-104, gemma.rs:131-135, phi3.rs:101-107, phi2.rs:99-101
 *   RmsNorm / LayerNorm  rai-nn/src/rms_norm.rs:18-22, gemma.rs:42-54, rai-nn/src/layer_norm.rs:32-42
 *   Linear / Embedding   rai-nn/src/linear.rs:59-69, rai-nn/src/embedding.rs:25-30
 *   activations          rai-core/src/hlops/activations.rs (silu, new_gelu), candle.rs:545-553 (rsqrt = 1/sqrt),
 *                        candle.rs:792-803 (softmax = max, sub, exp, sum, div)
 * Deviations shared with rai_cpu.py: grouped-query attention for qwen2 uses the gemma/phi3 form
 * (repeat each KV head), RoPE tables are float32, tied embeddings are honoured.
 *
 * Build: gcc -O2 -fopenmp -shared -fPIC -o librai_ref.so rai_ref.c -lm      (oracle/build_ref.py)
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

enum { ARCH_QWEN2 = 0, ARCH_PHI2 = 1, ARCH_PHI3 = 2, ARCH_GEMMA = 3 };
enum { ACT_SILU = 1, ACT_GELU_TANH = 2 };

typedef struct {
  int32_t arch, vocab, hidden, inter, layers, q_heads, kv_heads, head_dim, rot, act, max_pos;
  double theta, eps;
} ref_config;

/* One layer's tensors, [out, in] row-major as the checkpoint stores them; absent ones are NULL.
 * phi3's fused qkv_proj / gate_up_proj are given as their row ranges (narrow on the output == rows
 * of the weight); phi2's fc1 / fc2 ride in up / down. */
typedef struct {
  const float *ln1_w, *ln1_b, *ln2_w;
  const float *q_w, *q_b, *k_w, *k_b, *v_w, *v_b, *o_w, *o_b;
  const float *gate_w, *up_w, *up_b, *down_w, *down_b;
} ref_layer;

typedef struct {
  ref_config c;
  const float *embed, *norm_w, *norm_b, *head_w, *head_b;
  const ref_layer* L;
  float *sin_t, *cos_t;   /* [max_pos, rot/2] */
  float *k_cache, *v_cache; /* [layers][batch][kv_heads][max_pos][head_dim] */
  int32_t batch_cap, len; /* cached tokens per sequence */
} ref_model;

/* y[m, n] = sum_k x[m, k] * w[n, k] + b[n]   (Linear::fwd: x . W^T + b) */
static void linear(const float* x, const float* w, const float* b, float* y, int m, int n, int k) {
#pragma omp parallel for schedule(static)
  for (int j = 0; j < n; ++j) {
    const float* wr = w + (size_t)j * k;
    for (int i = 0; i < m; ++i) {
      const float* xr = x + (size_t)i * k;
      float acc = 0.f;
      for (int t = 0; t < k; ++t) acc += xr[t] * wr[t];
      y[(size_t)i * n + j] = b ? acc + b[j] : acc;
    }
  }
}

static void rms_norm(const float* x, const float* w, float eps, int one_plus, float* y, int rows, int h) {
  for (int r = 0; r < rows; ++r) {
    const float* xr = x + (size_t)r * h;
    float ss = 0.f;
    for (int i = 0; i < h; ++i) ss += xr[i] * xr[i];
    const float inv = 1.0f / sqrtf(ss / (float)h + eps); /* rsqrt is sqrt then recip in the reference's backend */
    for (int i = 0; i < h; ++i) y[(size_t)r * h + i] = xr[i] * inv * (one_plus ? 1.0f + w[i] : w[i]);
  }
}

static void layer_norm(const float* x, const float* w, const float* b, float eps, float* y, int rows, int h) {
  for (int r = 0; r < rows; ++r) {
    const float* xr = x + (size_t)r * h;
    float mean = 0.f;
    for (int i = 0; i < h; ++i) mean += xr[i];
    mean /= (float)h;
    float var = 0.f;
    for (int i = 0; i < h; ++i) var += (xr[i] - mean) * (xr[i] - mean);
    var /= (float)h;
    const float inv = 1.0f / sqrtf(var + eps);
    for (int i = 0; i < h; ++i) y[(size_t)r * h + i] = (xr[i] - mean) * inv * w[i] + b[i];
  }
}

static float act_apply(int act, float x) {
  if (act == ACT_SILU) return x * (1.0f / (1.0f + expf(-x)));
  /* new_gelu: 0.5 x (1 + tanh(sqrt(2/pi) (x + 0.044715 x^3))) */
  const float c = sqrtf(2.0f / 3.14159265358979323846f);
  return 0.5f * x * (1.0f + tanhf(c * (x + 0.044715f * x * x * x)));
}

static void rope_tables(ref_model* m) {
  const ref_config* c = &m->c;
  const int half = c->rot / 2;
  m->sin_t = (float*)malloc(sizeof(float) * (size_t)c->max_pos * half);
  m->cos_t = (float*)malloc(sizeof(float) * (size_t)c->max_pos * half);
  for (int j = 0; j < half; ++j) {
    const int i = 2 * j;
    float inv;
    if (c->arch == ARCH_PHI2) inv = 1.0f / powf((float)c->theta, (float)i / (float)c->rot);              /* f32 throughout */
    else if (c->arch == ARCH_PHI3) inv = (float)(1.0 / pow(c->theta, (double)i / (double)c->rot));       /* f64, then cast */
    else inv = 1.0f / (float)pow(c->theta, (double)i / (double)c->rot);                                  /* f64 power, f32 division */
    for (int p = 0; p < c->max_pos; ++p) {
      const float f = (float)p * inv;
      m->sin_t[(size_t)p * half + j] = sinf(f);
      m->cos_t[(size_t)p * half + j] = cosf(f);
    }
  }
}

/* x*cos + rotate_half(x)*sin on the first `rot` lanes of one head at position pos, in place */
static void rope_head(const ref_model* m, float* x, int pos) {
  const int rot = m->c.rot, half = rot / 2;
  const float* sn = m->sin_t + (size_t)pos * half;
  const float* cs = m->cos_t + (size_t)pos * half;
  for (int i = 0; i < half; ++i) {
    const float a = x[i], b = x[i + half];
    x[i] = a * cs[i] + (-b) * sn[i];
    x[i + half] = b * cs[i] + a * sn[i];
  }
}

ref_model* ref_create(const ref_config* c, const float* embed, const float* norm_w, const float* norm_b, const float* head_w,
                      const float* head_b, const ref_layer* layers, int32_t batch_cap) {
  ref_model* m = (ref_model*)calloc(1, sizeof(ref_model));
  m->c = *c;
  m->embed = embed; m->norm_w = norm_w; m->norm_b = norm_b; m->head_w = head_w; m->head_b = head_b;
  ref_layer* L = (ref_layer*)malloc(sizeof(ref_layer) * (size_t)c->layers);
  memcpy(L, layers, sizeof(ref_layer) * (size_t)c->layers);
  m->L = L;
  m->batch_cap = batch_cap;
  const size_t n = (size_t)c->layers * batch_cap * c->kv_heads * c->max_pos * c->head_dim;
  m->k_cache = (float*)calloc(n, sizeof(float));
  m->v_cache = (float*)calloc(n, sizeof(float));
  rope_tables(m);
  return m;
}

void ref_destroy(ref_model* m) {
  if (!m) return;
  free((void*)m->L); free(m->sin_t); free(m->cos_t); free(m->k_cache); free(m->v_cache); free(m);
}

void ref_clear_kv_cache(ref_model* m) { m->len = 0; }

static float* cache_row(const ref_model* m, float* base, int layer, int b, int kvh, int t) {
  const ref_config* c = &m->c;
  return base + ((((size_t)layer * m->batch_cap + b) * c->kv_heads + kvh) * c->max_pos + t) * c->head_dim;
}

/* attention of one layer: xn [B*S, H] -> out [B*S, H] (after the output projection) */
static void attention(ref_model* m, int layer, const float* xn, float* out, int B, int S, int offset) {
  const ref_config* c = &m->c;
  const ref_layer* w = &m->L[layer];
  const int H = c->hidden, nq = c->q_heads, nkv = c->kv_heads, d = c->head_dim, rows = B * S, T = offset + S;
  float* q = (float*)malloc(sizeof(float) * (size_t)rows * nq * d);
  float* k = (float*)malloc(sizeof(float) * (size_t)rows * nkv * d);
  float* v = (float*)malloc(sizeof(float) * (size_t)rows * nkv * d);
  float* o = (float*)malloc(sizeof(float) * (size_t)rows * nq * d);
  linear(xn, w->q_w, w->q_b, q, rows, nq * d, H);
  linear(xn, w->k_w, w->k_b, k, rows, nkv * d, H);
  linear(xn, w->v_w, w->v_b, v, rows, nkv * d, H);
  for (int b = 0; b < B; ++b)
    for (int s = 0; s < S; ++s) {
      const size_t r = (size_t)b * S + s;
      for (int h = 0; h < nq; ++h) rope_head(m, q + (r * nq + h) * d, offset + s);
      for (int h = 0; h < nkv; ++h) {
        rope_head(m, k + (r * nkv + h) * d, offset + s);
        memcpy(cache_row(m, m->k_cache, layer, b, h, offset + s), k + (r * nkv + h) * d, sizeof(float) * d); /* cat([prev, new], 2) */
        memcpy(cache_row(m, m->v_cache, layer, b, h, offset + s), v + (r * nkv + h) * d, sizeof(float) * d);
      }
    }
  const int rep = nq / nkv; /* repeat_kv: query head h reads KV head h / rep */
  /* phi3.rs:202 divides in f32; qwen2.rs:208, gemma.rs:241 and phi2.rs:173 compute 1/sqrt(d) in f64 and multiply an f32 tensor by it */
  const float scale = (c->arch == ARCH_PHI3) ? 1.0f / sqrtf((float)d) : (float)(1.0 / sqrt((double)d));
#pragma omp parallel for collapse(2) schedule(static)
  for (int b = 0; b < B; ++b)
    for (int h = 0; h < nq; ++h) {
      float* sc = (float*)malloc(sizeof(float) * (size_t)T);
      float* ks = (float*)malloc(sizeof(float) * (size_t)d);
      for (int s = 0; s < S; ++s) {
        const float* qr = q + (((size_t)b * S + s) * nq + h) * d;
        const int visible = (S > 1) ? offset + s + 1 : T; /* causal mask only when more than one query row */
        float mx = -INFINITY;
        for (int t = 0; t < T; ++t) {
          const float* kr = cache_row(m, m->k_cache, layer, b, h / rep, t);
          float acc = 0.f;
          if (c->arch == ARCH_PHI2) { /* the scale is folded into K^T before the product, phi2.rs:249-251 */
            for (int i = 0; i < d; ++i) ks[i] = kr[i] * scale;
            for (int i = 0; i < d; ++i) acc += qr[i] * ks[i];
          } else {
            for (int i = 0; i < d; ++i) acc += qr[i] * kr[i];
            acc *= scale;
          }
          if (t >= visible) acc = (c->arch == ARCH_PHI2) ? -INFINITY : acc + -INFINITY; /* where(mask, -inf, w) / w + mask */
          sc[t] = acc;
          if (acc > mx) mx = acc;
        }
        float sum = 0.f;
        for (int t = 0; t < T; ++t) { sc[t] = expf(sc[t] - mx); sum += sc[t]; }
        float* orow = o + (((size_t)b * S + s) * nq + h) * d;
        for (int i = 0; i < d; ++i) orow[i] = 0.f;
        for (int t = 0; t < T; ++t) {
          const float p = sc[t] / sum;
          const float* vr = cache_row(m, m->v_cache, layer, b, h / rep, t);
          for (int i = 0; i < d; ++i) orow[i] += p * vr[i];
        }
      }
      free(sc); free(ks);
    }
  linear(o, w->o_w, w->o_b, out, rows, H, nq * d); /* transpose(1,2) + reshape is the [row, head, lane] order already */
  free(q); free(k); free(v); free(o);
}

static void mlp(const ref_model* m, int layer, const float* xn, float* out, int rows) {
  const ref_config* c = &m->c;
  const ref_layer* w = &m->L[layer];
  const int H = c->hidden, I = c->inter;
  float* up = (float*)malloc(sizeof(float) * (size_t)rows * I);
  linear(xn, w->up_w, w->up_b, up, rows, I, H);
  if (w->gate_w) {
    float* gate = (float*)malloc(sizeof(float) * (size_t)rows * I);
    linear(xn, w->gate_w, NULL, gate, rows, I, H);
    /* qwen2/gemma: act(gate) * up; phi3: up * act(gate) -- the same product */
    for (size_t i = 0; i < (size_t)rows * I; ++i) up[i] = act_apply(c->act, gate[i]) * up[i];
    free(gate);
  } else {
    for (size_t i = 0; i < (size_t)rows * I; ++i) up[i] = act_apply(c->act, up[i]); /* phi2: fc2(act(fc1(x))) */
  }
  linear(up, w->down_w, w->down_b, out, rows, H, I);
  free(up);
}

/* tokens [B, S] at positions offset.. -> logits of the last position [B, vocab]; returns 0, or -1 on bad arguments */
int32_t ref_forward(ref_model* m, const int32_t* tokens, int32_t B, int32_t S, int32_t offset, float* logits) {
  const ref_config* c = &m->c;
  if (B < 1 || B > m->batch_cap || S < 1 || offset != m->len || offset + S > c->max_pos) return -1;
  const int H = c->hidden, rows = B * S;
  float* x = (float*)malloc(sizeof(float) * (size_t)rows * H);
  float* xn = (float*)malloc(sizeof(float) * (size_t)rows * H);
  float* a = (float*)malloc(sizeof(float) * (size_t)rows * H);
  float* f = (float*)malloc(sizeof(float) * (size_t)rows * H);
  const float emb_scale = sqrtf((float)H);
  for (int r = 0; r < rows; ++r) {
    const int id = tokens[r];
    if (id < 0 || id >= c->vocab) { free(x); free(xn); free(a); free(f); return -1; }
    for (int i = 0; i < H; ++i) {
      const float e = m->embed[(size_t)id * H + i];
      x[(size_t)r * H + i] = (c->arch == ARCH_GEMMA) ? e * emb_scale : e;
    }
  }
  const float eps = (float)c->eps;
  for (int l = 0; l < c->layers; ++l) {
    const ref_layer* w = &m->L[l];
    if (c->arch == ARCH_PHI2) {
      layer_norm(x, w->ln1_w, w->ln1_b, eps, xn, rows, H);
      attention(m, l, xn, a, B, S, offset);
      mlp(m, l, xn, f, rows);
      for (size_t i = 0; i < (size_t)rows * H; ++i) x[i] = a[i] + f[i] + x[i]; /* attn + mlp + residual */
    } else {
      const int one_plus = c->arch == ARCH_GEMMA;
      rms_norm(x, w->ln1_w, eps, one_plus, xn, rows, H);
      attention(m, l, xn, a, B, S, offset);
      for (size_t i = 0; i < (size_t)rows * H; ++i) x[i] = (c->arch == ARCH_PHI3) ? a[i] + x[i] : x[i] + a[i];
      rms_norm(x, w->ln2_w, eps, one_plus, xn, rows, H);
      mlp(m, l, xn, f, rows);
      for (size_t i = 0; i < (size_t)rows * H; ++i) x[i] = x[i] + f[i];
    }
  }
  /* last position only, final norm, lm_head (phi2 normalises every row first: the same numbers for the row kept) */
  float* last = (float*)malloc(sizeof(float) * (size_t)B * H);
  for (int b = 0; b < B; ++b) memcpy(last + (size_t)b * H, x + ((size_t)b * S + S - 1) * H, sizeof(float) * H);
  if (c->arch == ARCH_PHI2) layer_norm(last, m->norm_w, m->norm_b, eps, xn, B, H);
  else rms_norm(last, m->norm_w, eps, c->arch == ARCH_GEMMA, xn, B, H);
  linear(xn, m->head_w, m->head_b, logits, B, c->vocab, H);
  m->len = offset + S;
  free(x); free(xn); free(a); free(f); free(last);
  return 0;
}
