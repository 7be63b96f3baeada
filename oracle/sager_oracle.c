/*
 * sager_oracle.c - CPU restatement of SAGER's Q4_K MoE expert hot path.
 *
 * TEST INFRASTRUCTURE ONLY. This file is the parity checker for the CUDA
 * library: it may be called from tests/, from __graft_entry__.smoke() and from
 * bench.py's cpu_baseline / --impl reference legs. Nothing in the product
 * package (sager_b200/) may import, link or execute it.
 *
 * Each function restates one piece of the reference (paths are relative to
 * the samaidev/sager tree) and cites the lines it follows. Integer results
 * (Q8 codes, bsums, sub-block dots, routed indices, dispatch plan) are exact
 * by construction; fp32 results follow the reference's operation order but
 * are compiled with -ffp-contract=off, so they agree with a build of the
 * reference itself only to fp32 rounding (the reference is built with FMA
 * contraction enabled). Parity status: pinned against the reference's own
 * CPU code compiled from its sources (oracle/_ref) and against golden
 * vectors that build wrote (tests/golden/).
 *
 * Plain C99, no dependencies beyond libm and pthreads.
 */
#include <math.h>
#include <pthread.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define QK_K 256
#define QK 32
#define NSB 8
#define Q4K_BYTES 144
#define Q8K_BYTES 276

/* ---- block layouts: include/sager/kernels/q4_k.hpp:45-63 ------------------ */
#pragma pack(push, 1)
typedef struct {
  uint16_t d;
  uint16_t dmin;
  uint8_t scales[12];
  uint8_t qs[128];
} orc_q4k;
typedef struct {
  float d;
  int8_t qs[QK_K];
  int16_t bsums[NSB];
} orc_q8k;
#pragma pack(pop)

typedef char orc_assert_q4k[(sizeof(orc_q4k) == Q4K_BYTES) ? 1 : -1];
typedef char orc_assert_q8k[(sizeof(orc_q8k) == Q8K_BYTES) ? 1 : -1];

/* ---- fp16 helpers --------------------------------------------------------- */

/* Exact fp16 -> fp32 (same values as q4_k.hpp:66-91). */
float orc_half_to_float(uint16_t h) {
  const uint32_t sign = ((uint32_t)h & 0x8000u) << 16;
  const uint32_t exp = (h >> 10) & 0x1Fu;
  uint32_t man = h & 0x3FFu;
  uint32_t bits;
  if (exp == 0) {
    if (man == 0) {
      bits = sign;
    } else {
      int e = 0;
      while ((man & 0x400u) == 0) { man <<= 1; ++e; }
      bits = sign | ((uint32_t)(113 - e) << 23) | ((man & 0x3FFu) << 13);
    }
  } else if (exp == 0x1F) {
    bits = sign | 0x7F800000u | (man << 13);
  } else {
    bits = sign | ((exp + 112u) << 23) | (man << 13);
  }
  float f;
  memcpy(&f, &bits, 4);
  return f;
}

/* fp32 -> fp16, round to nearest even: what the device's __float2half does
 * (every fp16 store in moe.cu:13-15 and norm_rotary.cu goes through it). */
uint16_t orc_float_to_half_rn(float f) {
  uint32_t x;
  memcpy(&x, &f, 4);
  const uint32_t sign = (x >> 16) & 0x8000u;
  const uint32_t ax = x & 0x7FFFFFFFu;
  if (ax >= 0x7F800000u) {                       /* inf / nan */
    return (uint16_t)(sign | 0x7C00u | ((ax > 0x7F800000u) ? 0x200u : 0u));
  }
  if (ax >= 0x477FF000u) return (uint16_t)(sign | 0x7C00u);  /* rounds to inf */
  if (ax < 0x33000001u) return (uint16_t)sign;   /* <= 2^-25: rounds to zero */
  int e = (int)(ax >> 23) - 127;
  uint32_t m = (ax & 0x7FFFFFu) | 0x800000u;     /* 24-bit significand */
  int shift;
  uint32_t hexp;
  if (e < -14) { shift = 13 + (-14 - e); hexp = 0; }
  else         { shift = 13;             hexp = (uint32_t)(e + 15); }
  const uint32_t half_ulp = 1u << (shift - 1);
  const uint32_t rem = m & ((1u << shift) - 1u);
  uint32_t hm = m >> shift;
  if (rem > half_ulp || (rem == half_ulp && (hm & 1u))) ++hm;
  uint32_t out;
  if (hexp == 0) out = hm;                       /* subnormal; carry makes it normal */
  else out = ((hexp - 1u) << 10) + hm;           /* hm carries the implicit bit */
  return (uint16_t)(sign | out);
}

/* The reference's HOST helper truncates instead of rounding
 * (q4_k.hpp:93-108); its tests build fp16 inputs with it. */
uint16_t orc_float_to_half_trunc(float f) {
  uint32_t bits;
  memcpy(&bits, &f, 4);
  const uint32_t sign = (bits >> 16) & 0x8000u;
  const int32_t exp = (int32_t)((bits >> 23) & 0xFF) - 127 + 15;
  uint32_t man = bits & 0x7FFFFFu;
  if (exp >= 0x1F) return (uint16_t)(sign | 0x7C00u);
  if (exp <= 0) {
    if (exp < -10) return (uint16_t)sign;
    man |= 0x800000u;
    return (uint16_t)(sign | (man >> (14 - exp)));
  }
  return (uint16_t)(sign | ((uint32_t)exp << 10) | (man >> 13));
}

/* ---- 6-bit scale packing: q4_k.hpp:110-130 -------------------------------- */
void orc_get_scale_min_k4(int j, const uint8_t* q, uint8_t* d, uint8_t* m) {
  if (j < 4) {
    *d = q[j] & 63;
    *m = q[j + 4] & 63;
  } else {
    *d = (uint8_t)((q[j + 4] & 0xF) | ((q[j - 4] >> 6) << 4));
    *m = (uint8_t)((q[j + 4] >> 4) | ((q[j] >> 6) << 4));
  }
}

void orc_set_scale_min_k4(int j, uint8_t* q, uint8_t d, uint8_t m) {
  if (j < 4) {
    q[j] = (uint8_t)((q[j] & 0xC0) | (d & 63));
    q[j + 4] = (uint8_t)((q[j + 4] & 0xC0) | (m & 63));
  } else {
    q[j + 4] = (uint8_t)((d & 0xF) | ((m & 0xF) << 4));
    q[j - 4] = (uint8_t)((q[j - 4] & 0x3F) | ((d >> 4) << 6));
    q[j] = (uint8_t)((q[j] & 0x3F) | ((m >> 4) << 6));
  }
}

static void block_scales(const orc_q4k* b, float* sd, float* sm) {
  /* q4_avx2.cpp:30-39: sd = d*sc and sm = dmin*mn, each rounded to fp32. */
  const float d = orc_half_to_float(b->d);
  const float dmin = orc_half_to_float(b->dmin);
  for (int j = 0; j < NSB; ++j) {
    uint8_t d6, m6;
    orc_get_scale_min_k4(j, b->scales, &d6, &m6);
    sd[j] = d * (float)d6;
    sm[j] = dmin * (float)m6;
  }
}

/* ---- dequant: src/kernels/q4_k.cpp:13-42 ----------------------------------- */
void orc_dequant_row(const void* blocks, float* out, int n) {
  const orc_q4k* bl = (const orc_q4k*)blocks;
  const int nb = n / QK_K;
  for (int b = 0; b < nb; ++b) {
    float sd[NSB], sm[NSB];
    block_scales(&bl[b], sd, sm);
    float* ob = out + (size_t)b * QK_K;
    for (int s = 0; s < NSB; ++s) {
      const uint8_t* q = bl[b].qs + (s >> 1) * 32;
      for (int l = 0; l < QK; ++l) {
        const int nib = (s & 1) ? (q[l] >> 4) : (q[l] & 0xF);
        ob[s * QK + l] = sd[s] * (float)nib - sm[s];
      }
    }
  }
}

/* ---- Q8_K activation quantiser ---------------------------------------------
 * Host fp32 input: q4_k.cpp:44-61 and q4_avx2.cpp:77-94 (same arithmetic). */
void orc_quantize_row_q8k(const float* x, void* out, int n) {
  orc_q8k* ob = (orc_q8k*)out;
  const int nb = n / QK_K;
  for (int b = 0; b < nb; ++b) {
    const float* xb = x + (size_t)b * QK_K;
    float amax = 1e-30f;
    for (int i = 0; i < QK_K; ++i) amax = fmaxf(amax, fabsf(xb[i]));
    const float d = amax / 127.f;
    const float id = d > 0.f ? 1.f / d : 0.f;
    int sums[NSB] = {0};
    for (int i = 0; i < QK_K; ++i) {
      int q = (int)nearbyintf(xb[i] * id);
      q = q > 127 ? 127 : (q < -127 ? -127 : q);
      ob[b].qs[i] = (int8_t)q;
      sums[i >> 5] += q;
    }
    ob[b].d = d;
    for (int s = 0; s < NSB; ++s) ob[b].bsums[s] = (int16_t)sums[s];
  }
}

/* Device input is fp16 widened to fp32 first: q4_k.cu:94-130. The reference's
 * own test requires this to equal the host quantiser bit for bit on
 * fp16-representable inputs (tests/test_cuda_q4.cu:106-134). */
void orc_quantize_row_q8k_f16(const uint16_t* x16, void* out, int n) {
  float tmp[QK_K];
  const int nb = n / QK_K;
  for (int b = 0; b < nb; ++b) {
    for (int i = 0; i < QK_K; ++i) tmp[i] = orc_half_to_float(x16[(size_t)b * QK_K + i]);
    orc_quantize_row_q8k(tmp, (uint8_t*)out + (size_t)b * Q8K_BYTES, QK_K);
  }
}

/* ---- Q4_K weight quantiser ("M" flavour): q4_k.cpp:68-174 ------------------ */
static float q4_eval_err(const float* sb, float dd, float mm) {
  const float id = dd > 0.f ? 1.f / dd : 0.f;
  float err = 0.f;
  for (int j = 0; j < QK; ++j) {
    int q = (int)nearbyintf((sb[j] + mm) * id);
    q = q < 0 ? 0 : (q > 15 ? 15 : q);
    const float w = dd * (float)q - mm;
    const float e = sb[j] - w;
    err += e * e;
  }
  return err;
}

static int clampi(int v, int lo, int hi) { return v < lo ? lo : (v > hi ? hi : v); }

void orc_quantize_row_q4k(const float* x, void* out, int n) {
  orc_q4k* ob = (orc_q4k*)out;
  const int nb = n / QK_K;
  uint8_t codes[NSB][QK];
  for (int b = 0; b < nb; ++b) {
    const float* xb = x + (size_t)b * QK_K;
    orc_q4k* bl = &ob[b];
    memset(bl, 0, sizeof(*bl));
    memset(codes, 0, sizeof(codes));

    float max_abs = 1e-30f;   /* largest sub-block range */
    for (int s = 0; s < NSB; ++s) {
      float mn = xb[s * QK], mx = xb[s * QK];
      for (int j = 1; j < QK; ++j) {
        mn = fminf(mn, xb[s * QK + j]);
        mx = fmaxf(mx, xb[s * QK + j]);
      }
      max_abs = fmaxf(max_abs, mx - mn);
    }
    const float d = max_abs / 63.f;
    const float dmin = max_abs / 63.f;
    /* The block stores fp16(d) but the search below keeps using the fp32 d:
     * that is what the reference does (q4_k.cpp:103-106). */
    bl->d = orc_float_to_half_trunc(d);
    bl->dmin = orc_float_to_half_trunc(dmin);

    for (int s = 0; s < NSB; ++s) {
      const float* sb = xb + s * QK;
      float mn = sb[0], mx = sb[0];
      for (int j = 1; j < QK; ++j) { mn = fminf(mn, sb[j]); mx = fmaxf(mx, sb[j]); }
      if (mx == mn) { orc_set_scale_min_k4(s, bl->scales, 1, 0); continue; }

      const float d_ideal = (mx - mn) / 15.f;
      const int is_ideal = clampi((int)nearbyintf(d_ideal / d), 1, 63);
      const int im_ideal = clampi((int)nearbyintf(-mn / dmin), 0, 63);
      float best = q4_eval_err(sb, d * (float)is_ideal, dmin * (float)im_ideal);
      int b_is = is_ideal, b_im = im_ideal;
      const int is_hi = is_ideal + 16 < 63 ? is_ideal + 16 : 63;
      const int im_hi = im_ideal + 16 < 63 ? im_ideal + 16 : 63;
      for (int is = (is_ideal - 16 > 1 ? is_ideal - 16 : 1); is <= is_hi; is += 4) {
        for (int im = (im_ideal - 16 > 0 ? im_ideal - 16 : 0); im <= im_hi; im += 4) {
          const float err = q4_eval_err(sb, d * (float)is, dmin * (float)im);
          if (err < best) { best = err; b_is = is; b_im = im; }
        }
      }
      /* fine pass: the loop bounds re-read b_is / b_im as they move (as the reference's do) */
      for (int is = (b_is - 2 > 1 ? b_is - 2 : 1); is <= (b_is + 2 < 63 ? b_is + 2 : 63); ++is) {
        for (int im = (b_im - 2 > 0 ? b_im - 2 : 0); im <= (b_im + 2 < 63 ? b_im + 2 : 63); ++im) {
          const float err = q4_eval_err(sb, d * (float)is, dmin * (float)im);
          if (err < best) { best = err; b_is = is; b_im = im; }
        }
      }
      const float bd = d * (float)b_is;
      const float bm = dmin * (float)b_im;
      const float id = bd > 0.f ? 1.f / bd : 0.f;
      for (int j = 0; j < QK; ++j) {
        codes[s][j] = (uint8_t)clampi((int)nearbyintf((sb[j] + bm) * id), 0, 15);
      }
      orc_set_scale_min_k4(s, bl->scales, (uint8_t)b_is, (uint8_t)b_im);
    }
    for (int g = 0; g < NSB / 2; ++g) {
      uint8_t* q = bl->qs + g * 32;
      for (int l = 0; l < 32; ++l) {
        q[l] = (uint8_t)((codes[2 * g][l] & 0xF) | ((codes[2 * g + 1][l] & 0xF) << 4));
      }
    }
  }
}

/* ---- the bit-exact unit: one sub-block's int32 dot ---------------------------
 * q4_k.cu:38-53, q4_avx2.cpp:99-119, q4_k.cpp:195-199. Order-free. */
static int32_t subblock_dot(const orc_q4k* b, const orc_q8k* xb, int s) {
  const uint8_t* q = b->qs + (s >> 1) * 32;
  const int8_t* xq = xb->qs + s * QK;
  int32_t ip = 0;
  if (s & 1) { for (int l = 0; l < QK; ++l) ip += (int32_t)(q[l] >> 4) * xq[l]; }
  else       { for (int l = 0; l < QK; ++l) ip += (int32_t)(q[l] & 0xF) * xq[l]; }
  return ip;
}

/* out[(r*nb + blk)*8 + s] for every row, super-block and sub-block. */
void orc_subblock_dots(const void* w, const void* xq, int32_t* out, int n_rows, int k) {
  const orc_q4k* wb = (const orc_q4k*)w;
  const orc_q8k* xb = (const orc_q8k*)xq;
  const int nb = k / QK_K;
  for (int r = 0; r < n_rows; ++r)
    for (int blk = 0; blk < nb; ++blk)
      for (int s = 0; s < NSB; ++s)
        out[((size_t)r * nb + blk) * NSB + s] = subblock_dot(&wb[(size_t)r * nb + blk], &xb[blk], s);
}

/* Scalar reference dot: q4_k.cpp:176-207 (term by term into one accumulator). */
float orc_vec_dot_ref(const void* w, const void* xq, int n) {
  const orc_q4k* wb = (const orc_q4k*)w;
  const orc_q8k* xb = (const orc_q8k*)xq;
  const int nb = n / QK_K;
  float acc = 0.f;
  for (int b = 0; b < nb; ++b) {
    float sd[NSB], sm[NSB];
    block_scales(&wb[b], sd, sm);
    for (int s = 0; s < NSB; ++s) {
      const int32_t p = subblock_dot(&wb[b], &xb[b], s);
      acc += xb[b].d * (sd[s] * (float)p - sm[s] * (float)xb[b].bsums[s]);
    }
  }
  return acc;
}

/* CPU row accumulation: q4_avx2.cpp:124-145 (per block sum, then row acc). */
void orc_gemv_q4k_q8k(const void* w, const void* xq, float* y, int n_rows, int k) {
  const orc_q4k* wb = (const orc_q4k*)w;
  const orc_q8k* xb = (const orc_q8k*)xq;
  const int nb = k / QK_K;
  for (int r = 0; r < n_rows; ++r) {
    const orc_q4k* row = wb + (size_t)r * nb;
    float acc = 0.f;
    for (int blk = 0; blk < nb; ++blk) {
      float sd[NSB], sm[NSB];
      block_scales(&row[blk], sd, sm);
      float sum = 0.f;
      for (int s = 0; s < NSB; ++s) {
        const int32_t ip = subblock_dot(&row[blk], &xb[blk], s);
        sum += xb[blk].d * (sd[s] * (float)ip - sm[s] * (float)xb[blk].bsums[s]);
      }
      acc += sum;
    }
    y[r] = acc;
  }
}

/* Device row accumulation: q4_k.cu:57-91. Lane l sums the flat sub-blocks
 * g = l, l+32, ... ascending, then the shfl_down tree 16,8,4,2,1. */
static float shfl_down_tree(float* lane) {
  for (int off = 16; off > 0; off >>= 1)
    for (int l = 0; l < off; ++l) lane[l] = lane[l] + lane[l + off];
  return lane[0];
}

void orc_gemv_q4k_q8k_lane_order(const void* w, const void* xq, float* y, int n_rows, int k) {
  const orc_q4k* wb = (const orc_q4k*)w;
  const orc_q8k* xb = (const orc_q8k*)xq;
  const int nb = k / QK_K;
  const int nsg = nb * NSB;
  for (int r = 0; r < n_rows; ++r) {
    const orc_q4k* row = wb + (size_t)r * nb;
    float lane[32];
    for (int l = 0; l < 32; ++l) {
      float acc = 0.f;
      for (int g = l; g < nsg; g += 32) {
        const int blk = g >> 3, s = g & 7;
        float sd[NSB], sm[NSB];
        block_scales(&row[blk], sd, sm);
        const int32_t ip = subblock_dot(&row[blk], &xb[blk], s);
        acc += xb[blk].d * (sd[s] * (float)ip - sm[s] * (float)xb[blk].bsums[s]);
      }
      lane[l] = acc;
    }
    y[r] = shfl_down_tree(lane);
  }
}

/* ---- CPU expert FFN: q4_avx2.cpp:175-196 ----------------------------------- */
void orc_expert_ffn_q4(const void* w_gate, const void* w_up, const void* w_out,
                       const float* x, float* y, float* scratch, int hidden, int n_ff) {
  orc_q8k* xq = (orc_q8k*)malloc((size_t)(hidden / QK_K) * sizeof(orc_q8k));
  orc_q8k* hq = (orc_q8k*)malloc((size_t)(n_ff / QK_K) * sizeof(orc_q8k));
  orc_quantize_row_q8k(x, xq, hidden);
  float* g = scratch;
  float* u = scratch + n_ff;
  orc_gemv_q4k_q8k(w_gate, xq, g, n_ff, hidden);
  orc_gemv_q4k_q8k(w_up, xq, u, n_ff, hidden);
  for (int i = 0; i < n_ff; ++i) {
    const float gv = g[i];
    g[i] = gv / (1.f + expf(-gv)) * u[i];   /* std::exp on a float is expf */
  }
  orc_quantize_row_q8k(g, hq, n_ff);
  orc_gemv_q4k_q8k(w_out, hq, y, hidden, n_ff);
  free(xq);
  free(hq);
}

/* ---- router ------------------------------------------------------------------
 * Logits: q4_k.cu:133-149. acc += w*x is contracted to an FMA by nvcc, so the
 * restatement uses fmaf; lane-strided ascending i, then the shuffle tree. */
void orc_router_logits(const float* w, const uint16_t* x16, float* y, int n_rows, int k) {
  float* xf = (float*)malloc((size_t)k * sizeof(float));
  for (int i = 0; i < k; ++i) xf[i] = orc_half_to_float(x16[i]);
  for (int r = 0; r < n_rows; ++r) {
    const float* row = w + (size_t)r * k;
    float lane[32];
    for (int l = 0; l < 32; ++l) {
      float acc = 0.f;
      for (int i = l; i < k; i += 32) acc = fmaf(row[i], xf[i], acc);
      lane[l] = acc;
    }
    y[r] = shfl_down_tree(lane);
  }
  free(xf);
}

/* Softmax + greedy top-k on probabilities: moe.cu:25-85 (and :165-234,
 * mmq.cu:420-510). prob_scratch holds n_expert floats. Ties go to the lower
 * index, NaN is never picked, a pass with nothing valid yields kk % n_expert.
 * write_shared = 0 restates router_topk_fused, which leaves slot K alone. */
void orc_router_topk(const float* logits, int* idx, float* weight, int n_expert, int k,
                     float shared_w, int write_shared, float* prob) {
  float mx = -1e30f;
  for (int i = 0; i < n_expert; ++i) mx = fmaxf(mx, logits[i]);
  float z = 0.f;
  for (int i = 0; i < n_expert; ++i) z += expf(logits[i] - mx);
  for (int i = 0; i < n_expert; ++i) prob[i] = expf(logits[i] - mx) / z;
  float wsum = 0.f;
  for (int kk = 0; kk < k; ++kk) {
    float bv = -1.f;
    int bi = -1;
    for (int i = 0; i < n_expert; ++i) {
      const float p = prob[i];
      if (p == p && p > bv) { bv = p; bi = i; }   /* first strict max = lowest index on ties */
    }
    if (bi < 0) bi = kk % n_expert;
    prob[bi] = -1.f;
    idx[kk] = bi;
    weight[kk] = bv;
    wsum += bv;
  }
  if (wsum > 0.f) for (int kk = 0; kk < k; ++kk) weight[kk] /= wsum;
  if (write_shared) weight[k] = shared_w;
}

/* ---- device plan: moe.cu:366-434 -------------------------------------------
 * Position inside an expert is unspecified in the reference (atomics); this
 * restatement fills in ascending (row, kk) order. idx and weight rows have
 * stride k+1. */
void orc_dispatch_scan(const int* idx, float* weight, int* gslot, int* grows, int* off,
                       int* toff, int* meta, int n_rows, int k, int n_expert, int tok_per) {
  int* hist = (int*)calloc((size_t)n_expert, sizeof(int));
  int* fill = (int*)calloc((size_t)n_expert, sizeof(int));
  int bad = 0;
  for (int r = 0; r < n_rows; ++r) {
    for (int kk = 0; kk < k; ++kk) {
      const int e = idx[(size_t)r * (k + 1) + kk];
      if (e < 0 || e >= n_expert) {
        for (int q = 0; q <= k; ++q) weight[(size_t)r * (k + 1) + q] = 0.f;
        ++bad;
        continue;
      }
      ++hist[e];
    }
  }
  int acc = 0, tacc = 0;
  for (int e = 0; e < n_expert; ++e) {
    off[e] = acc;
    toff[e] = tacc;
    fill[e] = acc;
    acc += hist[e];
    tacc += (hist[e] + tok_per - 1) / tok_per;
  }
  off[n_expert] = acc;
  toff[n_expert] = tacc;
  meta[0] = acc;
  meta[1] = tacc;
  meta[2] = bad;
  for (int r = 0; r < n_rows; ++r) {
    for (int kk = 0; kk < k; ++kk) {
      const int e = idx[(size_t)r * (k + 1) + kk];
      if (e < 0 || e >= n_expert) { gslot[(size_t)r * k + kk] = -1; continue; }
      const int pos = fill[e]++;
      gslot[(size_t)r * k + kk] = pos;
      grows[pos] = r;
    }
  }
  free(hist);
  free(fill);
}

/* ---- SwiGLU on fp16 storage: norm_rotary.cu:133-141 ------------------------- */
void orc_silu_mul_f16(uint16_t* out, const uint16_t* g, const uint16_t* u, int total) {
  for (int i = 0; i < total; ++i) {
    const float gv = orc_half_to_float(g[i]);
    const float uv = orc_half_to_float(u[i]);
    out[i] = orc_float_to_half_rn(gv / (1.f + expf(-gv)) * uv);
  }
}

/* ---- combine: moe.cu:88-100 (idx < 0 skipped) and :265-280 (positional) ----- */
void orc_combine_f16(uint16_t* out, const uint16_t* expert_out, const int* idx,
                     const float* weight, int k, int hidden) {
  for (int i = 0; i < hidden; ++i) {
    float acc = orc_half_to_float(out[i]);
    for (int kk = 0; kk < k; ++kk) {
      if (idx[kk] < 0) continue;
      acc += weight[kk] * orc_half_to_float(expert_out[(size_t)kk * hidden + i]);
    }
    out[i] = orc_float_to_half_rn(acc);
  }
}

void orc_combine_batched_f16(uint16_t* out, const uint16_t* expert_y, const float* weight,
                             int n_used, int hidden, int n_rows) {
  for (int r = 0; r < n_rows; ++r) {
    const uint16_t* yrow = expert_y + (size_t)r * (n_used + 1) * hidden;
    const float* wrow = weight + (size_t)r * (n_used + 1);
    for (int i = 0; i < hidden; ++i) {
      float acc = orc_half_to_float(out[(size_t)r * hidden + i]);
      for (int kk = 0; kk < n_used + 1; ++kk)
        acc += wrow[kk] * orc_half_to_float(yrow[(size_t)kk * hidden + i]);
      out[(size_t)r * hidden + i] = orc_float_to_half_rn(acc);
    }
  }
}

/* ---- whole MoE layer, fp32 end to end ---------------------------------------
 * Router as the device computes it (logits from fp16 x, top-k on
 * probabilities), every selected expert and the shared expert through the CPU
 * FFN (expert_ffn_q4, which never applies router weights: contract C2 in
 * include/sager/core/expert_source.hpp:14-17), then the weighted sum in slot
 * order kk = 0..K with the shared expert in slot K (moe.cu:265-280), in fp32.
 *
 * x16        [n][H] fp16 activations (the fp32 FFN input is their exact widening)
 * router_w   [E][H] fp32
 * w_tab      [3][E] host pointers to gate / up / down matrices (NULL = absent:
 *            the expert contributes zero, as the device path does before the
 *            CPU patch, q4_k.cu:697-710)
 * shared     [3] pointers for the shared expert, or NULL entries for none
 * resid      [n][H] fp32 residual, may be NULL (zeros)
 * out        [n][H] fp32
 * out_idx    [n][K+1] ints, out_w [n][K+1] floats (slot K = shared_w)
 * n_threads  worker threads over (token, slot) FFN jobs
 */
typedef struct {
  const void *wg, *wu, *wd;
  const float* x;
  float* y;
  int hidden, n_ff;
} ffn_job;

typedef struct {
  ffn_job* jobs;
  int n_jobs;
  int next;
  pthread_mutex_t mu;
} ffn_queue;

static void* ffn_worker(void* arg) {
  ffn_queue* q = (ffn_queue*)arg;
  float* scratch = NULL;
  int scratch_ff = 0;
  for (;;) {
    pthread_mutex_lock(&q->mu);
    const int j = q->next < q->n_jobs ? q->next++ : -1;
    pthread_mutex_unlock(&q->mu);
    if (j < 0) break;
    ffn_job* jb = &q->jobs[j];
    if (jb->n_ff > scratch_ff) {
      free(scratch);
      scratch = (float*)malloc((size_t)2 * jb->n_ff * sizeof(float));
      scratch_ff = jb->n_ff;
    }
    orc_expert_ffn_q4(jb->wg, jb->wu, jb->wd, jb->x, jb->y, scratch, jb->hidden, jb->n_ff);
  }
  free(scratch);
  return NULL;
}

static void run_ffn_jobs(ffn_job* jobs, int n_jobs, int n_threads) {
  ffn_queue q;
  q.jobs = jobs;
  q.n_jobs = n_jobs;
  q.next = 0;
  pthread_mutex_init(&q.mu, NULL);
  if (n_threads <= 1) {
    ffn_worker(&q);
  } else {
    pthread_t* th = (pthread_t*)malloc((size_t)n_threads * sizeof(pthread_t));
    for (int t = 0; t < n_threads; ++t) pthread_create(&th[t], NULL, ffn_worker, &q);
    for (int t = 0; t < n_threads; ++t) pthread_join(th[t], NULL);
    free(th);
  }
  pthread_mutex_destroy(&q.mu);
}

void orc_moe_layer(const uint16_t* x16, const float* router_w, const void* const* w_tab,
                   const void* const* shared, const float* resid, float* out, int* out_idx,
                   float* out_w, float* out_logits, int n, int hidden, int n_ff,
                   int n_expert, int k, float shared_w, int n_threads) {
  const int slots = k + 1;
  float* xf = (float*)malloc((size_t)n * hidden * sizeof(float));
  float* ys = (float*)calloc((size_t)n * slots * hidden, sizeof(float));
  float* logits = (float*)malloc((size_t)n_expert * sizeof(float));
  float* prob = (float*)malloc((size_t)n_expert * sizeof(float));
  ffn_job* jobs = (ffn_job*)malloc((size_t)n * slots * sizeof(ffn_job));
  int n_jobs = 0;
  for (size_t i = 0; i < (size_t)n * hidden; ++i) xf[i] = orc_half_to_float(x16[i]);
  for (int r = 0; r < n; ++r) {
    orc_router_logits(router_w, x16 + (size_t)r * hidden, logits, n_expert, hidden);
    if (out_logits) memcpy(out_logits + (size_t)r * n_expert, logits, (size_t)n_expert * sizeof(float));
    orc_router_topk(logits, out_idx + (size_t)r * slots, out_w + (size_t)r * slots, n_expert, k,
                    shared_w, 1, prob);
    out_idx[(size_t)r * slots + k] = -1;
    for (int kk = 0; kk < slots; ++kk) {
      const void *wg, *wu, *wd;
      if (kk < k) {
        const int e = out_idx[(size_t)r * slots + kk];
        wg = w_tab[0 * n_expert + e];
        wu = w_tab[1 * n_expert + e];
        wd = w_tab[2 * n_expert + e];
      } else {
        wg = shared ? shared[0] : NULL;
        wu = shared ? shared[1] : NULL;
        wd = shared ? shared[2] : NULL;
      }
      if (!wg || !wu || !wd) continue;
      ffn_job* jb = &jobs[n_jobs++];
      jb->wg = wg; jb->wu = wu; jb->wd = wd;
      jb->x = xf + (size_t)r * hidden;
      jb->y = ys + ((size_t)r * slots + kk) * hidden;
      jb->hidden = hidden;
      jb->n_ff = n_ff;
    }
  }
  run_ffn_jobs(jobs, n_jobs, n_threads);
  for (int r = 0; r < n; ++r) {
    for (int i = 0; i < hidden; ++i) {
      float acc = resid ? resid[(size_t)r * hidden + i] : 0.f;
      for (int kk = 0; kk < slots; ++kk)
        acc += out_w[(size_t)r * slots + kk] * ys[((size_t)r * slots + kk) * hidden + i];
      out[(size_t)r * hidden + i] = acc;
    }
  }
  free(xf); free(ys); free(logits); free(prob); free(jobs);
}

/* Bare FFN jobs on a thread pool: the timed CPU baseline when the reference's
 * own pool (oracle/_ref) is not available. x [n_jobs][hidden], y likewise;
 * job j uses weights w3[3*j .. 3*j+2]. */
void orc_expert_ffn_batch(const void* const* w3, const float* x, float* y, int n_jobs,
                          int hidden, int n_ff, int n_threads) {
  ffn_job* jobs = (ffn_job*)malloc((size_t)n_jobs * sizeof(ffn_job));
  for (int j = 0; j < n_jobs; ++j) {
    jobs[j].wg = w3[3 * j]; jobs[j].wu = w3[3 * j + 1]; jobs[j].wd = w3[3 * j + 2];
    jobs[j].x = x + (size_t)j * hidden;
    jobs[j].y = y + (size_t)j * hidden;
    jobs[j].hidden = hidden;
    jobs[j].n_ff = n_ff;
  }
  run_ffn_jobs(jobs, n_jobs, n_threads);
  free(jobs);
}
