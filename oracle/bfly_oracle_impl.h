/* Test infrastructure, not product code: a plain-C restatement of the reference's
 * CPU algorithm for the butterfly multiply.  Included once per element type by
 * bfly_oracle.c with
 *   R    the real scalar type (float / double)
 *   NC   components per element (1 real, 2 complex: re, im interleaved)
 *   FN(x) the name-mangling macro for that instantiation
 *
 * Arithmetic follows the reference exactly: every product is rounded before the
 * sum (no FMA contraction; the file is built with -ffp-contract=off), complex
 * products are (ac - bd, ad + bc) as c10::complex computes them, and gradient
 * accumulation runs in the reference's loop order.
 */

/* out = a * b */
static inline void FN(mul)(const R *a, const R *b, R *out) {
#if NC == 1
  out[0] = a[0] * b[0];
#else
  R re = a[0] * b[0] - a[1] * b[1];
  R im = a[0] * b[1] + a[1] * b[0];
  out[0] = re;
  out[1] = im;
#endif
}

/* out = conj(a) */
static inline void FN(conj)(const R *a, R *out) {
  out[0] = a[0];
#if NC == 2
  out[1] = -a[1];
#endif
}

/* out = a*x + b*y  (two rounded products, then one add per component) */
static inline void FN(mul2add)(const R *a, const R *x, const R *b, const R *y, R *out) {
  R p[NC], q[NC];
  FN(mul)(a, x, p);
  FN(mul)(b, y, q);
  for (int c = 0; c < NC; ++c) out[c] = p[c] + q[c];
}

/* One radix-2 stage applied in place to `buf` (B,S,n), reading `src` instead of
 * `buf` when src != NULL (first stage: zero-padded read of the input).
 * Mirrors csrc/cpu/butterfly_cpu.cpp:38-57. */
static void FN(stage_fw)(const R *tw_stage_base, int64_t tw_stack_stride, const R *src,
                         int64_t src_B, int64_t src_S, int64_t src_size, const R *prev, R *dst,
                         int64_t B, int64_t S, int64_t n, int64_t stride) {
  for (int64_t b = 0; b < B; ++b) {
    for (int64_t s = 0; s < S; ++s) {
      const R *tw = tw_stage_base + s * tw_stack_stride;
      for (int64_t i = 0; i < n / 2; ++i) {
        int64_t low = i % stride;
        int64_t pos = 2 * (i - low) + low;
        const R *t = tw + i * 4 * NC; /* t00 t01 t10 t11 */
        R x0[NC], x1[NC];
        if (src) {
          for (int c = 0; c < NC; ++c) {
            x0[c] = pos < src_size ? src[(b * src_B + s * src_S + pos) * NC + c] : (R)0;
            x1[c] = pos + stride < src_size ? src[(b * src_B + s * src_S + pos + stride) * NC + c] : (R)0;
          }
        } else {
          for (int c = 0; c < NC; ++c) {
            x0[c] = prev[((b * S + s) * n + pos) * NC + c];
            x1[c] = prev[((b * S + s) * n + pos + stride) * NC + c];
          }
        }
        R y0[NC], y1[NC];
        FN(mul2add)(t + 0 * NC, x0, t + 1 * NC, x1, y0);
        FN(mul2add)(t + 2 * NC, x0, t + 3 * NC, x1, y1);
        for (int c = 0; c < NC; ++c) {
          dst[((b * S + s) * n + pos) * NC + c] = y0[c];
          dst[((b * S + s) * n + pos + stride) * NC + c] = y1[c];
        }
      }
    }
  }
}

/* Forward.  twiddle (S,nblocks,log_n,n/2,2,2) contiguous; x (B,S,input_size) with
 * element strides x_sB, x_sS (x_sS may be 0 for a stack-broadcast input);
 * out (B,S,output_size) contiguous.  Mirrors csrc/cpu/butterfly_cpu.cpp:17-66. */
int FN(bfly_oracle_fw)(const R *twiddle, const R *x, int64_t x_sB, int64_t x_sS, R *out, int64_t B,
                       int64_t S, int log_n, int nblocks, int64_t input_size, int64_t output_size,
                       int increasing_stride) {
  const int64_t n = (int64_t)1 << log_n;
  if (output_size > n || log_n < 1 || nblocks < 1) return -1;
  R *work = (R *)malloc(sizeof(R) * NC * (size_t)(B * S * n + 1));
  if (!work) return -2;
  const int64_t tw_stage = (n / 2) * 4 * NC;
  const int64_t tw_stack = (int64_t)nblocks * log_n * tw_stage;
  for (int block = 0; block < nblocks; ++block) {
    int cur_inc = (increasing_stride != 0) != (block % 2 != 0);
    for (int idx = 0; idx < log_n; ++idx) {
      int log_stride = cur_inc ? idx : (log_n - 1 - idx);
      const R *tws = twiddle + ((int64_t)block * log_n + idx) * tw_stage;
      int first = (block == 0 && idx == 0);
      FN(stage_fw)(tws, tw_stack, first ? x : NULL, x_sB, x_sS, input_size, work, work, B, S, n,
                   (int64_t)1 << log_stride);
    }
  }
  for (int64_t r = 0; r < B * S; ++r)
    memcpy(out + r * output_size * NC, work + r * n * NC, sizeof(R) * NC * (size_t)output_size);
  free(work);
  return 0;
}

/* Backward.  grad (B,S,output_size) contiguous; d_twiddle like twiddle (overwritten);
 * d_x (B,S,input_size) contiguous (columns >= n are zero).  Stores every stage
 * output like the reference does.  Mirrors csrc/cpu/butterfly_cpu.cpp:68-177. */
int FN(bfly_oracle_bw)(const R *twiddle, const R *x, int64_t x_sB, int64_t x_sS, const R *grad,
                       R *d_twiddle, R *d_x, int64_t B, int64_t S, int log_n, int nblocks,
                       int64_t input_size, int64_t output_size, int increasing_stride) {
  const int64_t n = (int64_t)1 << log_n;
  if (output_size > n || log_n < 1 || nblocks < 1) return -1;
  const int64_t L = (int64_t)nblocks * log_n;
  const int64_t plane = B * S * n * NC;
  R *store = (R *)malloc(sizeof(R) * (size_t)(plane * L + 1)); /* output of stage t at store + t*plane */
  R *g = (R *)malloc(sizeof(R) * (size_t)(plane + 1));
  if (!store || !g) { free(store); free(g); return -2; }
  const int64_t tw_stage = (n / 2) * 4 * NC;
  const int64_t tw_stack = (int64_t)nblocks * log_n * tw_stage;
  memset(d_twiddle, 0, sizeof(R) * (size_t)(S * tw_stack));
  /* forward, keeping every stage output except the last */
  for (int64_t t = 0; t < L - 1; ++t) {
    int block = (int)(t / log_n), idx = (int)(t % log_n);
    int cur_inc = (increasing_stride != 0) != (block % 2 != 0);
    int log_stride = cur_inc ? idx : (log_n - 1 - idx);
    const R *tws = twiddle + t * tw_stage;
    FN(stage_fw)(tws, tw_stack, t == 0 ? x : NULL, x_sB, x_sS, input_size,
                 t == 0 ? NULL : store + (t - 1) * plane, store + t * plane, B, S, n,
                 (int64_t)1 << log_stride);
  }
  /* backward sweep */
  for (int64_t t = L - 1; t >= 0; --t) {
    int block = (int)(t / log_n), idx = (int)(t % log_n);
    int cur_inc = (increasing_stride != 0) != (block % 2 != 0);
    int log_stride = cur_inc ? idx : (log_n - 1 - idx);
    int64_t stride = (int64_t)1 << log_stride;
    const R *prev = t == 0 ? NULL : store + (t - 1) * plane;
    for (int64_t b = 0; b < B; ++b) {
      for (int64_t s = 0; s < S; ++s) {
        const R *tw = twiddle + t * tw_stage + s * tw_stack;
        R *dtw = d_twiddle + t * tw_stage + s * tw_stack;
        for (int64_t i = 0; i < n / 2; ++i) {
          int64_t low = i % stride;
          int64_t pos = 2 * (i - low) + low;
          const R *tt = tw + i * 4 * NC;
          R g0[NC], g1[NC], x0[NC], x1[NC];
          for (int c = 0; c < NC; ++c) {
            if (t == L - 1) {
              g0[c] = pos < output_size ? grad[((b * S + s) * output_size + pos) * NC + c] : (R)0;
              g1[c] = pos + stride < output_size ? grad[((b * S + s) * output_size + pos + stride) * NC + c] : (R)0;
            } else {
              g0[c] = g[((b * S + s) * n + pos) * NC + c];
              g1[c] = g[((b * S + s) * n + pos + stride) * NC + c];
            }
            if (t == 0) {
              x0[c] = pos < input_size ? x[(b * x_sB + s * x_sS + pos) * NC + c] : (R)0;
              x1[c] = pos + stride < input_size ? x[(b * x_sB + s * x_sS + pos + stride) * NC + c] : (R)0;
            } else {
              x0[c] = prev[((b * S + s) * n + pos) * NC + c];
              x1[c] = prev[((b * S + s) * n + pos + stride) * NC + c];
            }
          }
          R c00[NC], c01[NC], c10[NC], c11[NC], o0[NC], o1[NC];
          FN(conj)(tt + 0 * NC, c00);
          FN(conj)(tt + 1 * NC, c01);
          FN(conj)(tt + 2 * NC, c10);
          FN(conj)(tt + 3 * NC, c11);
          FN(mul2add)(c00, g0, c10, g1, o0);
          FN(mul2add)(c01, g0, c11, g1, o1);
          for (int c = 0; c < NC; ++c) {
            g[((b * S + s) * n + pos) * NC + c] = o0[c];
            g[((b * S + s) * n + pos + stride) * NC + c] = o1[c];
          }
          R cx0[NC], cx1[NC], p[NC];
          FN(conj)(x0, cx0);
          FN(conj)(x1, cx1);
          R *d = dtw + i * 4 * NC;
          FN(mul)(g0, cx0, p); for (int c = 0; c < NC; ++c) d[0 * NC + c] += p[c];
          FN(mul)(g0, cx1, p); for (int c = 0; c < NC; ++c) d[1 * NC + c] += p[c];
          FN(mul)(g1, cx0, p); for (int c = 0; c < NC; ++c) d[2 * NC + c] += p[c];
          FN(mul)(g1, cx1, p); for (int c = 0; c < NC; ++c) d[3 * NC + c] += p[c];
        }
      }
    }
  }
  for (int64_t r = 0; r < B * S; ++r) {
    int64_t keep = input_size < n ? input_size : n;
    memcpy(d_x + r * input_size * NC, g + r * n * NC, sizeof(R) * NC * (size_t)keep);
    for (int64_t j = keep * NC; j < input_size * NC; ++j) d_x[r * input_size * NC + j] = (R)0;
  }
  free(store);
  free(g);
  return 0;
}

/* ---- base-4 (radix-4 stages, plus one radix-2 stage per block when log_n is odd) ----
 * Stage list of one block, in order (torch_butterfly/multiply_base4.py:23-40):
 *   idx = 0..log_n/2-1 : radix-4 on bits [b, b+2), b = cur_inc ? 2*idx : log_n-2-2*idx
 *   then, if log_n odd : radix-2 on bit  cur_inc ? log_n-1 : 0
 * twiddle4 (S,nblocks,log_n/2,n/4,4,4), twiddle2 (S,nblocks,log_n%2,n/2,2,2), contiguous. */

static void FN(stage4_fw)(const R *tw4_stage_base, int64_t tw4_stack_stride, const R *src, R *dst,
                          int64_t B, int64_t S, int64_t n, int64_t stride) {
  for (int64_t b = 0; b < B; ++b)
    for (int64_t s = 0; s < S; ++s) {
      const R *tw = tw4_stage_base + s * tw4_stack_stride;
      for (int64_t q = 0; q < n / 4; ++q) {
        int64_t k = q % stride, gidx = q / stride;
        int64_t base = gidx * 4 * stride + k;
        const R *t = tw + q * 16 * NC;
        R xin[4][NC], y[4][NC];
        for (int j = 0; j < 4; ++j)
          for (int c = 0; c < NC; ++c) xin[j][c] = src[((b * S + s) * n + base + j * stride) * NC + c];
        for (int i = 0; i < 4; ++i) {
          R acc[NC], p[NC];
          FN(mul)(t + (i * 4 + 0) * NC, xin[0], acc);
          for (int j = 1; j < 4; ++j) {
            FN(mul)(t + (i * 4 + j) * NC, xin[j], p);
            for (int c = 0; c < NC; ++c) acc[c] += p[c];
          }
          for (int c = 0; c < NC; ++c) y[i][c] = acc[c];
        }
        for (int i = 0; i < 4; ++i)
          for (int c = 0; c < NC; ++c) dst[((b * S + s) * n + base + i * stride) * NC + c] = y[i][c];
      }
    }
}

typedef struct { int radix; int log_stride; int64_t tw_off; } FN(b4stage);

static int FN(b4_plan)(int log_n, int nblocks, int inc, int64_t n, FN(b4stage) * st) {
  int cnt = 0;
  const int h = log_n / 2, odd = log_n % 2;
  for (int block = 0; block < nblocks; ++block) {
    int cur_inc = (inc != 0) != (block % 2 != 0);
    for (int idx = 0; idx < h; ++idx) {
      st[cnt].radix = 4;
      st[cnt].log_stride = cur_inc ? 2 * idx : log_n - 2 - 2 * idx;
      st[cnt].tw_off = ((int64_t)block * h + idx) * (n / 4) * 16 * NC;
      ++cnt;
    }
    if (odd) {
      st[cnt].radix = 2;
      st[cnt].log_stride = cur_inc ? log_n - 1 : 0;
      st[cnt].tw_off = (int64_t)block * (n / 2) * 4 * NC;
      ++cnt;
    }
  }
  return cnt;
}

int FN(bfly_oracle_base4_fw)(const R *twiddle4, const R *twiddle2, const R *x, int64_t x_sB,
                             int64_t x_sS, R *out, int64_t B, int64_t S, int log_n, int nblocks,
                             int64_t input_size, int64_t output_size, int increasing_stride) {
  const int64_t n = (int64_t)1 << log_n;
  if (output_size > n || log_n < 1 || nblocks < 1) return -1;
  const int h = log_n / 2, odd = log_n % 2;
  FN(b4stage) *st = (FN(b4stage) *)malloc(sizeof(FN(b4stage)) * (size_t)(nblocks * (h + 1) + 1));
  R *work = (R *)malloc(sizeof(R) * NC * (size_t)(B * S * n + 1));
  if (!st || !work) { free(st); free(work); return -2; }
  int cnt = FN(b4_plan)(log_n, nblocks, increasing_stride, n, st);
  const int64_t tw4_stack = (int64_t)nblocks * h * (n / 4) * 16 * NC;
  const int64_t tw2_stack = (int64_t)nblocks * odd * (n / 2) * 4 * NC;
  for (int64_t b = 0; b < B; ++b)
    for (int64_t s = 0; s < S; ++s)
      for (int64_t p = 0; p < n; ++p)
        for (int c = 0; c < NC; ++c)
          work[((b * S + s) * n + p) * NC + c] = p < input_size ? x[(b * x_sB + s * x_sS + p) * NC + c] : (R)0;
  for (int t = 0; t < cnt; ++t) {
    int64_t stride = (int64_t)1 << st[t].log_stride;
    if (st[t].radix == 4)
      FN(stage4_fw)(twiddle4 + st[t].tw_off, tw4_stack, work, work, B, S, n, stride);
    else
      FN(stage_fw)(twiddle2 + st[t].tw_off, tw2_stack, NULL, 0, 0, 0, work, work, B, S, n, stride);
  }
  for (int64_t r = 0; r < B * S; ++r)
    memcpy(out + r * output_size * NC, work + r * n * NC, sizeof(R) * NC * (size_t)output_size);
  free(work);
  free(st);
  return 0;
}

/* Base-4 backward: the adjoint of the forward above (the reference has no
 * hand-written base-4 backward; autograd of multiply_base4.py:7-41 defines it).
 *   dx_j = sum_i conj(T[i][j]) g_i ,  dT[i][j] += g_i conj(x_j)  summed over batch. */
int FN(bfly_oracle_base4_bw)(const R *twiddle4, const R *twiddle2, const R *x, int64_t x_sB,
                             int64_t x_sS, const R *grad, R *d_twiddle4, R *d_twiddle2, R *d_x,
                             int64_t B, int64_t S, int log_n, int nblocks, int64_t input_size,
                             int64_t output_size, int increasing_stride) {
  const int64_t n = (int64_t)1 << log_n;
  if (output_size > n || log_n < 1 || nblocks < 1) return -1;
  const int h = log_n / 2, odd = log_n % 2;
  FN(b4stage) *st = (FN(b4stage) *)malloc(sizeof(FN(b4stage)) * (size_t)(nblocks * (h + 1) + 1));
  if (!st) return -2;
  int cnt = FN(b4_plan)(log_n, nblocks, increasing_stride, n, st);
  const int64_t plane = B * S * n * NC;
  R *store = (R *)malloc(sizeof(R) * (size_t)(plane * cnt + 1)); /* input of stage t at store + t*plane */
  R *g = (R *)malloc(sizeof(R) * (size_t)(plane + 1));
  if (!store || !g) { free(st); free(store); free(g); return -2; }
  const int64_t tw4_stack = (int64_t)nblocks * h * (n / 4) * 16 * NC;
  const int64_t tw2_stack = (int64_t)nblocks * odd * (n / 2) * 4 * NC;
  memset(d_twiddle4, 0, sizeof(R) * (size_t)(S * tw4_stack));
  if (tw2_stack) memset(d_twiddle2, 0, sizeof(R) * (size_t)(S * tw2_stack));
  for (int64_t b = 0; b < B; ++b)
    for (int64_t s = 0; s < S; ++s)
      for (int64_t p = 0; p < n; ++p)
        for (int c = 0; c < NC; ++c) {
          store[((b * S + s) * n + p) * NC + c] = p < input_size ? x[(b * x_sB + s * x_sS + p) * NC + c] : (R)0;
          g[((b * S + s) * n + p) * NC + c] = p < output_size ? grad[((b * S + s) * output_size + p) * NC + c] : (R)0;
        }
  for (int t = 0; t < cnt - 1; ++t) {
    int64_t stride = (int64_t)1 << st[t].log_stride;
    if (st[t].radix == 4)
      FN(stage4_fw)(twiddle4 + st[t].tw_off, tw4_stack, store + t * plane, store + (t + 1) * plane, B, S, n, stride);
    else
      FN(stage_fw)(twiddle2 + st[t].tw_off, tw2_stack, NULL, 0, 0, 0, store + t * plane, store + (t + 1) * plane, B, S, n, stride);
  }
  for (int t = cnt - 1; t >= 0; --t) {
    int64_t stride = (int64_t)1 << st[t].log_stride;
    const R *xin = store + t * plane;
    const int r = st[t].radix;
    const int64_t nun = n / r;
    for (int64_t b = 0; b < B; ++b)
      for (int64_t s = 0; s < S; ++s) {
        const R *tw = (r == 4 ? twiddle4 + s * tw4_stack : twiddle2 + s * tw2_stack) + st[t].tw_off;
        R *dtw = (r == 4 ? d_twiddle4 + s * tw4_stack : d_twiddle2 + s * tw2_stack) + st[t].tw_off;
        for (int64_t q = 0; q < nun; ++q) {
          int64_t k = q % stride, gidx = q / stride;
          int64_t base = gidx * r * stride + k;
          const R *tt = tw + q * r * r * NC;
          R *dd = dtw + q * r * r * NC;
          R gi[4][NC], xj[4][NC], o[4][NC];
          for (int j = 0; j < r; ++j)
            for (int c = 0; c < NC; ++c) {
              gi[j][c] = g[((b * S + s) * n + base + j * stride) * NC + c];
              xj[j][c] = xin[((b * S + s) * n + base + j * stride) * NC + c];
            }
          for (int j = 0; j < r; ++j) {
            R acc[NC], p[NC], ct[NC];
            FN(conj)(tt + (0 * r + j) * NC, ct);
            FN(mul)(ct, gi[0], acc);
            for (int i = 1; i < r; ++i) {
              FN(conj)(tt + (i * r + j) * NC, ct);
              FN(mul)(ct, gi[i], p);
              for (int c = 0; c < NC; ++c) acc[c] += p[c];
            }
            for (int c = 0; c < NC; ++c) o[j][c] = acc[c];
          }
          for (int i = 0; i < r; ++i)
            for (int j = 0; j < r; ++j) {
              R cx[NC], p[NC];
              FN(conj)(xj[j], cx);
              FN(mul)(gi[i], cx, p);
              for (int c = 0; c < NC; ++c) dd[(i * r + j) * NC + c] += p[c];
            }
          for (int j = 0; j < r; ++j)
            for (int c = 0; c < NC; ++c) g[((b * S + s) * n + base + j * stride) * NC + c] = o[j][c];
        }
      }
  }
  for (int64_t rr = 0; rr < B * S; ++rr) {
    int64_t keep = input_size < n ? input_size : n;
    memcpy(d_x + rr * input_size * NC, g + rr * n * NC, sizeof(R) * NC * (size_t)keep);
    for (int64_t j = keep * NC; j < input_size * NC; ++j) d_x[rr * input_size * NC + j] = (R)0;
  }
  free(st);
  free(store);
  free(g);
  return 0;
}
