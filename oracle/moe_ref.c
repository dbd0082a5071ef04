/* CPU checker for the FP8 block-scaled routed-MoE layer, plain C + OpenMP.
 * TEST INFRASTRUCTURE ONLY: tests, the smoke check and the benchmark's
 * cpu_baseline / reference arm load this library; nothing that ships may.
 *
 * It restates the same reference files as moe_ref.py (paths inside the
 * reference project):
 *   router logits   tools/benchmark/export_qwen36_router_bf16_capture.py:78
 *   top-8 / renorm  third-party SGLang fused_topk (not in the reference tree)
 *   shared slot     runtime/gfx950/routing/decode/qwen36_shared_gate_append_bridge.h:10-23
 *   token sort      scripts/rocm/integrations/sglang/netra_gfx1151_sglang.py:1186-1209
 *   FP8 quantiser   harness/gfx950/fp8/moe/decode/qwen36_moe_silu_mul_quant_fp8_gfx950.hip:57-94
 *   gate_up / down  tools/benchmark/export_qwen36_moe_stage1_capture.py:80-97,
 *                   tools/benchmark/export_qwen36_moe_stage2_capture.py:90-110
 *   SiLU*up         kernels/gfx950/templates/moe/decode/silu_quant.inc:54-131
 * PARITY UNPINNED for the numeric path (the reference ships no golden vectors
 * for it); this file is pinned against moe_ref.py, which carries the pins that
 * do exist.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

enum { H = 2048, I = 512, NE = 256, TOPK = 8, SLOTS = 9, BLK = 128 };

static float e4m3_lut[256];
static int lut_ready = 0;

static float u2f(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }
static uint32_t f2u(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }
static float bf16_to_f32(uint16_t b) { return u2f((uint32_t)b << 16); }
static uint16_t f32_to_bf16(float f) {
  uint32_t u = f2u(f);
  return (uint16_t)((u + 0x7fffu + ((u >> 16) & 1u)) >> 16);
}
/* FP64 -> BF16 with a single rounding: below 2^-126 -> signed zero, 2^128 and above -> infinity, NaN stays NaN. */
static uint16_t f64_to_bf16(double d) {
  uint64_t u; memcpy(&u, &d, 8);
  uint16_t sign = (uint16_t)((u >> 63) << 15);
  int64_t mag = (int64_t)(u & 0x7fffffffffffffffULL);
  if (mag > 0x7ff0000000000000LL) return (uint16_t)(sign | 0x7fc0u);
  int64_t r = (mag + ((1LL << 44) - 1) + ((mag >> 45) & 1)) >> 45;
  r -= (896LL << 7);
  if (r < (1 << 7)) r = 0;
  if (r > 0x7f80) r = 0x7f80;
  return (uint16_t)(sign | (uint16_t)r);
}

static void init_lut(void) {
  if (lut_ready) return;
  for (int c = 0; c < 256; ++c) {
    int e = (c >> 3) & 15, m = c & 7;
    float v = e == 0 ? ldexpf((float)m / 8.0f, -6) : ldexpf(1.0f + (float)m / 8.0f, e - 7);
    if ((c & 0x7f) == 0x7f) v = NAN;
    e4m3_lut[c] = (c & 0x80) ? -v : v;
  }
  lut_ready = 1;
}

/* FP32 -> E4M3 code, round-to-nearest-even, saturating at 448. */
static uint8_t e4m3_encode(float x) {
  uint8_t sign = (f2u(x) >> 31) ? 0x80 : 0;
  float a = fabsf(x);
  if (a != a) return 0x7f;
  if (a > 448.0f) a = 448.0f;
  int ex; frexpf(a, &ex);
  int e = ex - 1; if (e < -6 || a == 0.0f) e = -6;
  float step = ldexpf(1.0f, e - 3);
  float q = nearbyintf(a / step);           /* default rounding mode = half to even */
  float v = q * step;
  if (v < ldexpf(1.0f, -6)) return sign | (uint8_t)(v * 512.0f);
  int ex2; float m = frexpf(v, &ex2);       /* v = m * 2^ex2, m in [0.5,1) */
  int e2 = ex2 - 1;
  int mant = (int)((m * 2.0f - 1.0f) * 8.0f);
  return sign | (uint8_t)(((e2 + 7) << 3) + mant);
}

int moe_ref_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

/* torchrun exports OMP_NUM_THREADS=1; callers that time this library set the thread count themselves */
void moe_ref_set_threads(int n) {
#ifdef _OPENMP
  if (n > 0) omp_set_num_threads(n);
#else
  (void)n;
#endif
}

uint8_t moe_ref_e4m3_encode(float x) { return e4m3_encode(x); }

/* per-128 quantiser: x FP32 [rows, cols] -> codes [rows, cols], scales [rows, cols/128] */
static void quant_row(const float* x, int cols, uint8_t* q, float* s) {
  const float inv448 = u2f(0x3b124925u), floor_ = u2f(0x2edbe6ffu);
  for (int g = 0; g < cols / BLK; ++g) {
    float amax = floor_;
    for (int i = 0; i < BLK; ++i) amax = fmaxf(amax, fabsf(x[g * BLK + i]));
    float scale = amax * inv448;
    float inv = 1.0f / scale;
    s[g] = scale;
    for (int i = 0; i < BLK; ++i) q[g * BLK + i] = e4m3_encode(x[g * BLK + i] * inv);
  }
}

void moe_ref_quant_fp8(const float* x, int rows, int cols, uint8_t* q, float* s) {
  init_lut();
#pragma omp parallel for schedule(static)
  for (int r = 0; r < rows; ++r) quant_row(x + (size_t)r * cols, cols, q + (size_t)r * cols, s + (size_t)r * (cols / BLK));
}

/* exact-dot router logits, BF16 bits [T, NE] */
void moe_ref_router_logits(const uint16_t* hidden, const uint16_t* rw, int T, uint16_t* logits) {
  double* w = (double*)malloc(sizeof(double) * NE * H);
  for (int i = 0; i < NE * H; ++i) w[i] = bf16_to_f32(rw[i]);
#pragma omp parallel for schedule(static)
  for (int t = 0; t < T; ++t) {
    double h[H];
    for (int k = 0; k < H; ++k) h[k] = bf16_to_f32(hidden[(size_t)t * H + k]);
    for (int e = 0; e < NE; ++e) {
      double acc[4] = {0, 0, 0, 0};
      const double* we = w + (size_t)e * H;
      for (int k = 0; k < H; k += 4) {
        acc[0] += h[k] * we[k]; acc[1] += h[k + 1] * we[k + 1];
        acc[2] += h[k + 2] * we[k + 2]; acc[3] += h[k + 3] * we[k + 3];
      }
      logits[(size_t)t * NE + e] = f64_to_bf16((acc[0] + acc[1]) + (acc[2] + acc[3]));
    }
  }
  free(w);
}

/* softmax / top-8 (logit desc, id asc) / renormalise; appends the shared slot */
void moe_ref_route_topk(const uint16_t* logits, const float* bias, const float* shared_w, int T,
                        int32_t* ids9, float* w9) {
#pragma omp parallel for schedule(static)
  for (int t = 0; t < T; ++t) {
    float z[NE], p[NE];
    float zmax = -INFINITY;
    for (int e = 0; e < NE; ++e) {
      z[e] = bf16_to_f32(logits[(size_t)t * NE + e]);
      if (bias) z[e] = z[e] + bias[e];
      zmax = fmaxf(zmax, z[e]);
    }
    float denom = 0.0f;
    for (int e = 0; e < NE; ++e) { p[e] = expf(z[e] - zmax); denom += p[e]; }
    uint8_t taken[NE]; memset(taken, 0, sizeof taken);
    float sel[TOPK]; float s = 0.0f;
    for (int k = 0; k < TOPK; ++k) {
      int best = -1;
      for (int e = 0; e < NE; ++e)
        if (!taken[e] && (best < 0 || z[e] > z[best])) best = e;   /* strict > keeps lowest id */
      taken[best] = 1;
      ids9[t * SLOTS + k] = best;
      sel[k] = p[best] / denom;
      s += sel[k];
    }
    for (int k = 0; k < TOPK; ++k) w9[t * SLOTS + k] = sel[k] / s;
    ids9[t * SLOTS + TOPK] = NE;
    w9[t * SLOTS + TOPK] = shared_w ? shared_w[t] : 1.0f;
  }
}

/* stable expert-major order of the T*8 routed pairs */
void moe_ref_sort(const int32_t* ids9, int T, int32_t* perm, int32_t* counts, int32_t* offsets) {
  memset(counts, 0, sizeof(int32_t) * NE);
  for (int t = 0; t < T; ++t)
    for (int k = 0; k < TOPK; ++k) counts[ids9[t * SLOTS + k]]++;
  offsets[0] = 0;
  for (int e = 0; e < NE; ++e) offsets[e + 1] = offsets[e] + counts[e];
  int32_t* cur = (int32_t*)malloc(sizeof(int32_t) * NE);
  memcpy(cur, offsets, sizeof(int32_t) * NE);
  for (int t = 0; t < T; ++t)
    for (int k = 0; k < TOPK; ++k) perm[cur[ids9[t * SLOTS + k]]++] = t * TOPK + k;
  free(cur);
}

/* dequantise a [n, k] FP8 slab with 128x128 scales into FP32 */
static void dequant_slab(const uint8_t* q, const float* s, int n, int k, float* out) {
  int kb_n = k / BLK;
  for (int r = 0; r < n; ++r)
    for (int kb = 0; kb < kb_n; ++kb) {
      float sc = s[(r / BLK) * kb_n + kb];
      const uint8_t* src = q + (size_t)r * k + kb * BLK;
      float* dst = out + (size_t)r * k + kb * BLK;
      for (int i = 0; i < BLK; ++i) dst[i] = e4m3_lut[src[i]] * sc;
    }
}

/* out[n] = sum over K-blocks (ascending) of dot(a_deq[kb], w_deq[n, kb]); 8 partial lanes per block */
static void blockscale_matvec(const float* a_deq, const float* w_deq, int n, int k, float* out) {
  for (int r = 0; r < n; ++r) {
    const float* w = w_deq + (size_t)r * k;
    float acc = 0.0f;
    for (int kb = 0; kb < k / BLK; ++kb) {
      float l[8] = {0, 0, 0, 0, 0, 0, 0, 0};
      const float* aa = a_deq + kb * BLK; const float* ww = w + kb * BLK;
      for (int i = 0; i < BLK; i += 8)
        for (int j = 0; j < 8; ++j) l[j] += aa[i + j] * ww[i + j];
      acc += ((l[0] + l[1]) + (l[2] + l[3])) + ((l[4] + l[5]) + (l[6] + l[7]));
    }
    out[r] = acc;
  }
}

/* one (token row, expert) pair: FP8 hidden row -> FP32 down output [H]; also the
 * requantised intermediate when hq/hs are given */
static void expert_row(const uint8_t* aq, const float* as, const float* w13_deq, const float* w2_deq,
                       float* down, uint8_t* hq_out, float* hs_out) {
  float a_deq[H], gu[2 * I], h[I], h_deq[I], hs[I / BLK]; uint8_t hq[I];
  for (int k = 0; k < H; ++k) a_deq[k] = e4m3_lut[aq[k]] * as[k / BLK];
  blockscale_matvec(a_deq, w13_deq, 2 * I, H, gu);
  for (int i = 0; i < I; ++i) {
    float g = gu[i], u = gu[I + i];
    float sig = 1.0f / (1.0f + expf(-g));
    h[i] = bf16_to_f32(f32_to_bf16((g * sig) * u));
  }
  quant_row(h, I, hq, hs);
  for (int i = 0; i < I; ++i) h_deq[i] = e4m3_lut[hq[i]] * hs[i / BLK];
  blockscale_matvec(h_deq, w2_deq, H, I, down);
  if (hq_out) { memcpy(hq_out, hq, I); memcpy(hs_out, hs, sizeof hs); }
}

/* Whole layer.  n_slabs = routed experts + 1 (the last slab is the shared expert).
 * Outputs: logits bf16 [T,256], ids9/w9 [T,9], perm [T*8], counts [256], offsets [257],
 * a_fp8 [T,2048], a_scale [T,16], h_fp8 [T,9,512], h_scale [T,9,4] (either may be NULL),
 * out bf16 [T,2048]. */
int moe_ref_layer(const uint16_t* hidden, const uint16_t* router_w, const float* bias,
                  const float* shared_w, const uint8_t* w13, const float* w13_s,
                  const uint8_t* w2, const float* w2_s, int T,
                  uint16_t* logits, int32_t* ids9, float* w9, int32_t* perm, int32_t* counts,
                  int32_t* offsets, uint8_t* a_fp8, float* a_scale, uint8_t* h_fp8, float* h_scale,
                  uint16_t* out) {
  init_lut();
  moe_ref_router_logits(hidden, router_w, T, logits);
  moe_ref_route_topk(logits, bias, shared_w, T, ids9, w9);
  moe_ref_sort(ids9, T, perm, counts, offsets);
  float* hf = (float*)malloc(sizeof(float) * (size_t)T * H);
  for (size_t i = 0; i < (size_t)T * H; ++i) hf[i] = bf16_to_f32(hidden[i]);
  moe_ref_quant_fp8(hf, T, H, a_fp8, a_scale);
  free(hf);
  float* down = (float*)malloc(sizeof(float) * (size_t)T * SLOTS * H);
  if (!down) return -1;
  /* work items: each routed expert with rows, then the shared slab split into token chunks */
  const int chunk = 16;
  int shared_items = (T + chunk - 1) / chunk;
#pragma omp parallel
  {
    float* w13_deq = (float*)malloc(sizeof(float) * 2 * I * H);
    float* w2_deq = (float*)malloc(sizeof(float) * H * I);
#pragma omp for schedule(dynamic, 1)
    for (int item = 0; item < NE + shared_items; ++item) {
      int e = item < NE ? item : NE;
      int lo, hi;
      if (item < NE) { lo = offsets[e]; hi = offsets[e + 1]; }
      else { lo = (item - NE) * chunk; hi = lo + chunk < T ? lo + chunk : T; }
      if (hi <= lo) continue;
      dequant_slab(w13 + (size_t)e * 2 * I * H, w13_s + (size_t)e * (2 * I / BLK) * (H / BLK), 2 * I, H, w13_deq);
      dequant_slab(w2 + (size_t)e * H * I, w2_s + (size_t)e * (H / BLK) * (I / BLK), H, I, w2_deq);
      for (int r = lo; r < hi; ++r) {
        int t = item < NE ? perm[r] / TOPK : r;
        int s = item < NE ? perm[r] % TOPK : TOPK;
        size_t row = (size_t)t * SLOTS + s;
        expert_row(a_fp8 + (size_t)t * H, a_scale + (size_t)t * (H / BLK), w13_deq, w2_deq,
                   down + row * H, h_fp8 ? h_fp8 + row * I : NULL, h_scale ? h_scale + row * (I / BLK) : NULL);
      }
    }
    free(w13_deq); free(w2_deq);
  }
#pragma omp parallel for schedule(static)
  for (int t = 0; t < T; ++t)
    for (int n = 0; n < H; ++n) {
      float acc = 0.0f;
      for (int s = 0; s < SLOTS; ++s) acc += down[((size_t)t * SLOTS + s) * H + n] * w9[t * SLOTS + s];
      out[(size_t)t * H + n] = f32_to_bf16(acc);
    }
  free(down);
  return 0;
}
