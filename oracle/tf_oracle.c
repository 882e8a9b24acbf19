/* TEST INFRASTRUCTURE ONLY -- CPU restatement (plain C) of the fused
 * sparse-dense chains of SwiftWare-Lab/tile-fusion and of the inspectors that
 * schedule them.  Only tests/, the smoke check and bench.py's CPU-baseline leg
 * may load the library built from this file; the product path never does.
 *
 * Parity status: PINNED for the inspectors (I1-I4), the fused SpMM-SpMM
 * executor and the fused GeMM-SpMM executor -- tests compare every function
 * below with the reference's own code compiled in place (oracle/_ref) and with
 * the golden vectors that run produced (tests/golden/).  UNPINNED for
 * SDDMM-SpMM and the 2-layer GCN forward: the reference holds no C++
 * implementation of either; they follow the Python definitions cited below
 * and are cross-checked against the fp64 variants in this file.
 *
 * Each function cites the reference file:line it restates (paths are inside
 * the reference project).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

/* ------------------------------------------------------------------ */
/* small int vector                                                    */
/* ------------------------------------------------------------------ */
typedef struct { int *d; size_t n, cap; } ivec;
static void iv_init(ivec *v) { v->d = NULL; v->n = 0; v->cap = 0; }
static void iv_push(ivec *v, int x) {
  if (v->n == v->cap) {
    v->cap = v->cap ? v->cap * 2 : 64;
    v->d = (int *)realloc(v->d, v->cap * sizeof(int));
  }
  v->d[v->n++] = x;
}
static void iv_free(ivec *v) { free(v->d); v->d = NULL; v->n = v->cap = 0; }
static int cmp_int(const void *a, const void *b) {
  int x = *(const int *)a, y = *(const int *)b;
  return (x > y) - (x < y);
}

/* ------------------------------------------------------------------ */
/* schedule container: sym_lib::MultiDimensionalSet                    */
/*   fusion/include/sparse-fusion/MultiDimensionalSet.h:15-25          */
/* ------------------------------------------------------------------ */
typedef struct {
  int n1;        /* number of levels (wavefronts)                       */
  int n_parts;   /* ptr1[n1]                                            */
  int n_ids;     /* ptr2[n_parts]                                       */
  int has_ker;   /* ker_begin present ("Separated" packing)             */
  int *ptr1, *ptr2, *id, *type, *ker;
  double stats[8]; /* fused nodes, fused nnz, tile mean, tile std, #parts */
} orc_sched;

void orc_sched_dims(const orc_sched *s, int *n1, int *n_parts, int *n_ids, int *has_ker) {
  *n1 = s->n1; *n_parts = s->n_parts; *n_ids = s->n_ids; *has_ker = s->has_ker;
}
void orc_sched_copy(const orc_sched *s, int *ptr1, int *ptr2, int *id, int *type, int *ker,
                    double *stats) {
  memcpy(ptr1, s->ptr1, sizeof(int) * (s->n1 + 1));
  memcpy(ptr2, s->ptr2, sizeof(int) * (s->n_parts + 1));
  memcpy(id, s->id, sizeof(int) * s->n_ids);
  memcpy(type, s->type, sizeof(int) * s->n_ids);
  if (ker && s->has_ker) memcpy(ker, s->ker, sizeof(int) * 2 * s->n_parts);
  if (stats) memcpy(stats, s->stats, sizeof(s->stats));
}
void orc_sched_free(orc_sched *s) {
  if (!s) return;
  free(s->ptr1); free(s->ptr2); free(s->id); free(s->type); free(s->ker); free(s);
}

/* getNumberOfFusedNodes / getFusedNnzNum: fusion/src/MultiDimensionalSet.cpp:240-267 */
static void fused_counts(orc_sched *s, const int *Ap) {
  int fused = 0, fnnz = 0;
  if (s->n1 > 0)
    for (int j = s->ptr1[0]; j < s->ptr1[1]; ++j)
      for (int k = s->ptr2[j]; k < s->ptr2[j + 1]; ++k)
        if (s->type[k] == 1) { fused++; fnnz += Ap[s->id[k] + 1] - Ap[s->id[k]]; }
  s->stats[0] = fused; s->stats[1] = fnnz; s->stats[4] = s->n_parts;
}

/* ------------------------------------------------------------------ */
/* I1: fixed tiles.                                                    */
/*  SparseFusionInspector::generateFusedScheduleForAllFused            */
/*    fusion/include/sparse-fusion/Fusion_Inspector.h:32-55            */
/*  LBC consecutive branch        fusion/src/Fusion_Utils.cpp:510-548  */
/*  partitionByWeight             fusion/src/Fusion_Utils.cpp:365-388  */
/*  pairing / forward_pairing     fusion/src/SparseFusion.cpp:47-142,  */
/*                                fusion/src/Fusion_Utils.cpp:316-350  */
/*  separated packing             fusion/src/MultiDimensionalSet.cpp:124-185 */
/* ------------------------------------------------------------------ */
/* unit weights: even = ceil(n / parts); part i takes items until its count reaches even */
static void partition_by_unit_weight(int n, int parts, int *idx /* parts+1 */) {
  double even = ceil((double)n / parts);
  int j = 0;
  idx[0] = 0;
  for (int i = 0; i < parts; ++i) {
    double w = 0;
    while (w < even && j < n) { w += 1.0; j++; }
    idx[i + 1] = j;
  }
}

orc_sched *orc_inspect_fixed(int m, const int *Ap, const int *Ai, int threads, int iter_per_part) {
  int P = m / iter_per_part;
  if (P < 2 * threads) P = 2 * threads;
  int *pp = (int *)malloc(sizeof(int) * (P + 1));
  partition_by_unit_weight(m, P, pp);
  /* loop-1 rows fused into their own part iff every column is in the part */
  ivec *fused = (ivec *)malloc(sizeof(ivec) * P);
  char *visited = (char *)calloc(m, 1);
  for (int p = 0; p < P; ++p) {
    iv_init(&fused[p]);
    int lo = pp[p], hi = pp[p + 1];
    for (int r = lo; r < hi; ++r) {
      int ok = 1;
      for (int j = Ap[r]; j < Ap[r + 1]; ++j)
        if (Ai[j] < lo || Ai[j] >= hi) { ok = 0; break; }
      if (ok) { iv_push(&fused[p], r); visited[r] = 1; }
    }
  }
  ivec unv; iv_init(&unv);
  for (int r = 0; r < m; ++r) if (!visited[r]) iv_push(&unv, r);
  int u = (int)unv.n;
  int *up = NULL;
  if (u > 0) { up = (int *)malloc(sizeof(int) * (P + 1)); partition_by_unit_weight(u, P, up); }

  orc_sched *s = (orc_sched *)calloc(1, sizeof(orc_sched));
  s->n1 = u > 0 ? 2 : 1;
  s->n_parts = u > 0 ? 2 * P : P;
  s->has_ker = 1;
  s->ptr1 = (int *)calloc(s->n1 + 1, sizeof(int));
  s->ptr2 = (int *)calloc(s->n_parts + 1, sizeof(int));
  s->ker = (int *)calloc(2 * (size_t)s->n_parts, sizeof(int));
  size_t total = (size_t)m;
  for (int p = 0; p < P; ++p) total += fused[p].n;
  total += u;
  s->id = (int *)malloc(sizeof(int) * (total ? total : 1));
  s->type = (int *)malloc(sizeof(int) * (total ? total : 1));
  int cnt = 0, w = 0;
  for (int p = 0; p < P; ++p) {
    for (int r = pp[p]; r < pp[p + 1]; ++r) { s->id[cnt] = r; s->type[cnt] = 0; cnt++; }
    s->ker[2 * w] = cnt;
    for (size_t k = 0; k < fused[p].n; ++k) { s->id[cnt] = fused[p].d[k]; s->type[cnt] = 1; cnt++; }
    s->ker[2 * w + 1] = cnt;
    s->ptr2[++w] = cnt;
  }
  s->ptr1[1] = w;
  if (u > 0) {
    for (int p = 0; p < P; ++p) {
      s->ker[2 * w] = cnt; /* loop-0 list empty */
      for (int k = up[p]; k < up[p + 1]; ++k) { s->id[cnt] = unv.d[k]; s->type[cnt] = 1; cnt++; }
      s->ker[2 * w + 1] = cnt;
      s->ptr2[++w] = cnt;
    }
    s->ptr1[2] = w;
  }
  s->n_ids = cnt;
  fused_counts(s, Ap);
  for (int p = 0; p < P; ++p) iv_free(&fused[p]);
  free(fused); free(visited); free(pp); free(up); iv_free(&unv);
  return s;
}

/* ------------------------------------------------------------------ */
/* I2 / I3 / I4: variable tiles.                                       */
/*   InspectorForTileFusedCSRVariableTileSize                          */
/*     fusion/include/sparse-fusion/Fusion_Inspector.h:507-1052        */
/* ------------------------------------------------------------------ */
typedef struct vtile {
  int start, end;
  ivec fused;
  struct vtile *next;
} vtile;
static vtile *vt_new(int s, int e) {
  vtile *t = (vtile *)malloc(sizeof(vtile));
  t->start = s; t->end = e; t->next = NULL; iv_init(&t->fused);
  return t;
}
/* cost models, all in wrapping 32-bit int arithmetic as in :1020-1031 */
static int32_t wrap32(int64_t x) { return (int32_t)(uint32_t)(uint64_t)x; }
static int ws_spmm(int nnz, int uniq, int bcol, int tile, int fused, int ds) {
  int32_t a = wrap32((int64_t)uniq * bcol);
  int32_t b = wrap32((int64_t)tile * bcol);
  int32_t c = wrap32((int64_t)fused * bcol);
  int32_t s = wrap32((int64_t)nnz + a);
  s = wrap32((int64_t)s + b);
  s = wrap32((int64_t)s + c);
  s = wrap32((int64_t)s * ds);
  return wrap32((int64_t)s + wrap32((int64_t)nnz * 4));
}
static int ws_gemm(int fnnz, int bcol, int ccol, int tile, int fused, int ds) {
  int32_t s = wrap32((int64_t)tile * ccol);
  s = wrap32((int64_t)s + wrap32((int64_t)ccol * bcol));
  s = wrap32((int64_t)s + wrap32((int64_t)tile * bcol));
  s = wrap32((int64_t)s + wrap32((int64_t)fused * ccol));
  s = wrap32((int64_t)s + fnnz);
  s = wrap32((int64_t)s * ds);
  return wrap32((int64_t)s + wrap32((int64_t)fnnz * 4));
}
static int uniq_cols_range(const int *Ai, int lo, int hi, int *stamp, int *epoch) {
  int c = 0;
  (*epoch)++;
  for (int j = lo; j < hi; ++j)
    if (stamp[Ai[j]] != *epoch) { stamp[Ai[j]] = *epoch; c++; }
  return c;
}
static int fused_nnz(const vtile *t, const int *Ap) {
  int s = 0;
  for (size_t i = 0; i < t->fused.n; ++i) s += Ap[t->fused.d[i] + 1] - Ap[t->fused.d[i]];
  return s;
}
/* tile statistics: extractTilesSizeData :1034-1050 (float arithmetic) */
static void tile_stats(vtile *head, double *mean_out, double *std_out) {
  size_t n = 0; double acc = 0.0;
  for (vtile *c = head->next; c; c = c->next) { acc += (double)(c->end - c->start); n++; }
  float average = (float)(acc / (double)n);
  float var = 0;
  for (vtile *c = head->next; c; c = c->next) {
    int ts = c->end - c->start;
    var += (ts - average) * (ts - average);
  }
  var /= n;
  float sd = (float)sqrt(var);
  *mean_out = average; *std_out = sd;
}

/* kind 2: ...ForBothWavefronts(ACsr, BCol, DataSize)           :676-846
 * kind 3: ...GeMMSpMM(ACsr, BCol, CCol, DataSize)              :851-1017
 * kind 4: generateVariableTileSizeSchedule(ACsr, BCol, DataSize) :542-674
 * Returns NULL when the reference would divide by zero (initial tile 0). */
orc_sched *orc_inspect_variable(int kind, int m, const int *Ap, const int *Ai, int threads, int tile_m,
                                int bcol, int ccol, int ds) {
  int cache = tile_m;
  int min_max = 0, init;
  if (kind == 2) { min_max = m / (2 * threads); init = 4096 < min_max ? 4096 : min_max; }
  else if (kind == 3) { init = (tile_m / ds - bcol * ccol) / (bcol + ccol); if (init > m) init = m; }
  else { init = 4096 < m ? 4096 : m; }
  if (init <= 0) return NULL;
  int extra = m % init, removed = 0, ntiles = m / init;
  int per = (int)ceil(extra / (double)ntiles);
  vtile *head = vt_new(0, 0), *cur = head;
  for (int i = 0; i < ntiles; ++i) {
    int st = init * i + removed, en = st + init;
    if (extra > removed) {
      int ext = extra - removed < per ? extra - removed : per;
      en += ext; removed += ext;
    }
    cur->next = vt_new(st, en); cur = cur->next;
  }
  ivec unf; iv_init(&unf);
  if (kind == 4) {
    /* :576-590 -- every row is tested against every tile, first hit wins */
    for (int i = 0; i < m; ++i) {
      int ok = 0;
      for (cur = head->next; cur; cur = cur->next)
        if (Ai[Ap[i]] >= cur->start && Ai[Ap[i + 1] - 1] < cur->end) { iv_push(&cur->fused, i); ok = 1; break; }
      if (!ok) iv_push(&unf, i);
    }
  } else {
    for (cur = head->next; cur; cur = cur->next)
      for (int i = cur->start; i < cur->end; ++i) {
        if (Ai[Ap[i]] >= cur->start && Ai[Ap[i + 1] - 1] < cur->end) iv_push(&cur->fused, i);
        else iv_push(&unf, i);
      }
  }
  int *stamp = (int *)calloc(m > 0 ? m : 1, sizeof(int));
  int epoch = 0;
  /* shrink pass */
  cur = head;
  while (cur->next) {
    vtile *prev = cur;
    cur = cur->next;
    int ts = cur->end - cur->start, ws;
    if (kind == 3) ws = ws_gemm(fused_nnz(cur, Ap), bcol, ccol, ts, (int)cur->fused.n, ds);
    else {
      int nnz = Ap[cur->end] - Ap[cur->start];
      int uq = uniq_cols_range(Ai, Ap[cur->start], Ap[cur->end], stamp, &epoch);
      ws = ws_spmm(nnz, uq, bcol, ts, (int)cur->fused.n, ds);
    }
    if (ws > cache && ts > 1) {
      int sep = ts / 2 + cur->start;
      vtile *a = vt_new(cur->start, sep), *b = vt_new(sep, cur->end);
      for (size_t k = 0; k < cur->fused.n; ++k) {
        int fi = cur->fused.d[k];
        if (Ai[Ap[fi + 1] - 1] < sep) iv_push(&a->fused, fi);
        else if (Ai[Ap[fi]] >= sep) iv_push(&b->fused, fi);
        else iv_push(&unf, fi);
      }
      a->next = b; b->next = cur->next; prev->next = a;
      ntiles++;
      iv_free(&cur->fused); free(cur);
      cur = prev;
    }
  }
  /* wave 2 */
  ivec ufptr; iv_init(&ufptr);
  int n_uf_tiles;
  int u = (int)unf.n;
  int unf_per_part = 0;
  if (kind == 4) {
    /* :645-657: unsorted list split evenly over `threads` parts (float ceil) */
    unf_per_part = (int)ceilf(u / (float)threads);
    n_uf_tiles = threads;
  } else {
    qsort(unf.d, unf.n, sizeof(int), cmp_int);
    int stride = 16, nnz = 0, uft = 0, size = 0, uq = 0;
    epoch++;
    iv_push(&ufptr, 0);
    while (uft < u) {
      if (stride == 0) { /* the reference loops forever here (tiny m / many threads) */
        iv_free(&unf); iv_free(&ufptr); free(stamp);
        cur = head;
        while (cur) { vtile *t = cur; cur = cur->next; iv_free(&t->fused); free(t); }
        return NULL;
      }
      int lim = u < uft + stride ? u : uft + stride;
      for (int ii = uft; ii < lim; ++ii) {
        int row = unf.d[ii];
        for (int j = Ap[row]; j < Ap[row + 1]; ++j)
          if (stamp[Ai[j]] != epoch) { stamp[Ai[j]] = epoch; uq++; }
        nnz += Ap[row + 1] - Ap[row];
        size++;
      }
      int ws = ws_spmm(nnz, uq, bcol, size, 0, ds);
      int grow = (kind == 2) ? (((ws < cache) || (size == 1)) && (size + stride < min_max))
                             : ((ws < cache) || (size <= 16));
      if (grow) uft += stride;
      else {
        iv_push(&ufptr, uft);
        nnz = 0; uq = 0; epoch++;
        if (size <= stride) stride = stride / 2;
        if (size >= 3 * stride) stride = stride * 2;
        size = 0;
      }
    }
    iv_push(&ufptr, u);
    n_uf_tiles = (int)ufptr.n - 1;
  }
  orc_sched *s = (orc_sched *)calloc(1, sizeof(orc_sched));
  s->n1 = 2;
  s->n_parts = ntiles + n_uf_tiles;
  s->has_ker = kind != 4;
  s->ptr1 = (int *)calloc(3, sizeof(int));
  s->ptr1[1] = ntiles; s->ptr1[2] = ntiles + n_uf_tiles;
  s->ptr2 = (int *)calloc((size_t)s->n_parts + 1, sizeof(int));
  s->ker = s->has_ker ? (int *)calloc(2 * (size_t)s->n_parts, sizeof(int)) : NULL;
  s->id = (int *)malloc(sizeof(int) * 2 * (size_t)(m > 0 ? m : 1));
  s->type = (int *)malloc(sizeof(int) * 2 * (size_t)(m > 0 ? m : 1));
  int cnt = 0, pc = 0;
  for (cur = head->next; cur; cur = cur->next) {
    for (int j = cur->start; j < cur->end; ++j) { s->id[cnt] = j; s->type[cnt] = 0; cnt++; }
    if (s->ker) s->ker[2 * pc] = cnt;
    for (size_t k = 0; k < cur->fused.n; ++k) { s->id[cnt] = cur->fused.d[k]; s->type[cnt] = 1; cnt++; }
    if (s->ker) s->ker[2 * pc + 1] = cnt;
    s->ptr2[++pc] = cnt;
  }
  tile_stats(head, &s->stats[2], &s->stats[3]);
  for (int i = ntiles; i < ntiles + n_uf_tiles; ++i) {
    int p = i - ntiles, lo, hi;
    if (kind == 4) {
      lo = p * unf_per_part;
      hi = (p + 1) * unf_per_part < u ? (p + 1) * unf_per_part : u;
    } else { lo = ufptr.d[p]; hi = ufptr.d[p + 1]; }
    if (s->ker) s->ker[2 * i] = cnt;
    for (int j = lo; j < hi; ++j) { s->id[cnt] = unf.d[j]; s->type[cnt] = 1; cnt++; }
    if (s->ker) s->ker[2 * i + 1] = cnt;
    s->ptr2[i + 1] = cnt;
  }
  s->n_ids = cnt;
  fused_counts(s, Ap);
  cur = head;
  while (cur) { vtile *t = cur; cur = cur->next; iv_free(&t->fused); free(t); }
  iv_free(&unf); iv_free(&ufptr); free(stamp);
  return s;
}

/* ------------------------------------------------------------------ */
/* Executors (fp32, fused multiply-add chained in CSR order, which is  */
/* what the AVX2 reference kernels do per output element).             */
/* ------------------------------------------------------------------ */
/* spmmCsrSequential<float>  fusion/src/SpMM_SpMM.cpp:20-31 ; accumulates into Cx */
void orc_spmm_csr(int m, int n, const int *Ap, const int *Ai, const float *Ax, const float *Bx,
                  float *Cx) {
#pragma omp parallel for schedule(static)
  for (int i = 0; i < m; ++i)
    for (int j = Ap[i]; j < Ap[i + 1]; ++j) {
      const float *b = Bx + (size_t)Ai[j] * n;
      float *c = Cx + (size_t)i * n, a = Ax[j];
      for (int k = 0; k < n; ++k) c[k] = fmaf(a, b[k], c[k]);
    }
}

/* spmmCsrSpmmCsrFused<float>  fusion/src/SpMM_SpMM.cpp:211-248 and
 * spmmCsrSpmmCsrFusedVectorized2_32SP  fusion/src/SpMM_SpMM_vectorized.cpp:876-989.
 * D = A * (B * C) with A the second (outer) operator and B the first -- the
 * reference names the first operator "A" and the second "B"; here `P*` is the
 * producer operator (type 0 rows) and `Q*` the consumer operator (type 1 rows).
 * AC and D accumulate, the caller zeroes them. */
void orc_spmm_spmm_fused(int m, int n, const int *Pp, const int *Pi, const float *Px, const int *Qp,
                         const int *Qi, const float *Qx, const float *Cx, float *Dx, float *ACx,
                         int level_no, const int *level_ptr, const int *par_ptr, const int *partition,
                         const int *par_type) {
  (void)m;
  for (int l = 0; l < level_no; ++l) {
#pragma omp parallel for schedule(dynamic, 1)
    for (int w = level_ptr[l]; w < level_ptr[l + 1]; ++w)
      for (int k1 = par_ptr[w]; k1 < par_ptr[w + 1]; ++k1) {
        int i = partition[k1];
        if (par_type[k1] == 0) {
          float *o = ACx + (size_t)i * n;
          for (int j = Pp[i]; j < Pp[i + 1]; ++j) {
            const float *c = Cx + (size_t)Pi[j] * n; float a = Px[j];
            for (int k = 0; k < n; ++k) o[k] = fmaf(a, c[k], o[k]);
          }
        } else {
          float *o = Dx + (size_t)i * n;
          for (int j = Qp[i]; j < Qp[i + 1]; ++j) {
            const float *c = ACx + (size_t)Qi[j] * n; float a = Qx[j];
            for (int k = 0; k < n; ++k) o[k] = fmaf(a, c[k], o[k]);
          }
        }
      }
  }
}

/* forwardForOneLayerFusedParallelSeparatedVectorizedSP
 *   fusion/gcn/GCN_Layer_MKL_Forward_Utils.h:218-291 (weight [K x N], NoTrans) and the
 * scalar sibling :182-216 (weight [N x K], Trans; selected with w_transposed = 1).
 * Per tile: Tmp[tile rows] = Feat[tile rows] * W (beta = 0), then the fused rows
 * Out[i] += A[i,j] * Tmp[col_j].  The tile GEMM here sums over k in order with FMA;
 * MKL's own order is unspecified, so GEMM results are pinned to tolerance only. */
void orc_gemm_spmm_fused(int m, const int *Ap, const int *Ai, const float *Ax, int kdim, int n,
                         const float *feat, const float *w, int w_transposed, float *out, float *tmp,
                         int level_no, const int *level_ptr, const int *par_ptr, const int *mix_ptr,
                         const int *partition) {
  (void)m;
  for (int l = 0; l < level_no; ++l) {
#pragma omp parallel for schedule(dynamic, 1)
    for (int j1 = level_ptr[l]; j1 < level_ptr[l + 1]; ++j1) {
      int kb = par_ptr[j1], ke1 = mix_ptr[2 * j1], ke2 = mix_ptr[2 * j1 + 1];
      int ts = ke1 - kb;
      if (ts > 0) {
        int r0 = partition[kb];
        for (int r = r0; r < r0 + ts; ++r) {
          const float *f = feat + (size_t)r * kdim;
          float *t = tmp + (size_t)r * n;
          for (int c = 0; c < n; ++c) {
            float acc = 0.f;
            if (w_transposed) for (int k = 0; k < kdim; ++k) acc = fmaf(f[k], w[(size_t)c * kdim + k], acc);
            else for (int k = 0; k < kdim; ++k) acc = fmaf(f[k], w[(size_t)k * n + c], acc);
            t[c] = acc;
          }
        }
      }
      for (int k1 = ke1; k1 < ke2; ++k1) {
        int i = partition[k1];
        float *o = out + (size_t)i * n;
        for (int j = Ap[i]; j < Ap[i + 1]; ++j) {
          const float *t = tmp + (size_t)Ai[j] * n; float a = Ax[j];
          for (int c = 0; c < n; ++c) o[c] = fmaf(a, t[c], o[c]);
        }
      }
    }
  }
}

/* SDDMM-SpMM.  SDDMM semantics from sddmm_cpu, codegen/triton/sddmm.py:173-184:
 *   S[p] = A.data[p] * dot(Q[row(p)], K[col(p)]);  then D = S * V as a CSR SpMM
 * (fusion/src/SpMM_SpMM.cpp:20-31).  S is optional output (nnz floats) or NULL. */
void orc_sddmm_spmm(int m, const int *Ap, const int *Ai, const float *Ax, int kq, int nv,
                    const float *Q, const float *K, const float *V, float *S, float *D) {
#pragma omp parallel for schedule(dynamic, 64)
  for (int i = 0; i < m; ++i) {
    float *o = D + (size_t)i * nv;
    for (int c = 0; c < nv; ++c) o[c] = 0.f;
    const float *q = Q + (size_t)i * kq;
    for (int p = Ap[i]; p < Ap[i + 1]; ++p) {
      const float *kk = K + (size_t)Ai[p] * kq;
      float dot = 0.f;
      for (int t = 0; t < kq; ++t) dot = fmaf(q[t], kk[t], dot);
      float s = dot * Ax[p];
      if (S) S[p] = s;
      const float *v = V + (size_t)Ai[p] * nv;
      for (int c = 0; c < nv; ++c) o[c] = fmaf(s, v[c], o[c]);
    }
  }
}

/* One GCN layer as the torch binding computes it: out = A * (X * W^T), W stored
 * [out_dim x in_dim]  (binding-project/src/Functions.cpp:629-711,
 * binding-project/gcn-e2e-training/FusedGCNLayer.py:10-11), optional ReLU
 * (binding-project/gcn-e2e-training/FusedGCNModule.py:14-18).  tmp is m x out_dim. */
void orc_gcn_layer(int m, const int *Ap, const int *Ai, const float *Ax, int in_dim, int out_dim,
                   const float *X, const float *W, int relu, float *tmp, float *out) {
#pragma omp parallel for schedule(static)
  for (int r = 0; r < m; ++r) {
    const float *f = X + (size_t)r * in_dim;
    float *t = tmp + (size_t)r * out_dim;
    for (int c = 0; c < out_dim; ++c) {
      float acc = 0.f;
      for (int k = 0; k < in_dim; ++k) acc = fmaf(f[k], W[(size_t)c * in_dim + k], acc);
      t[c] = acc;
    }
  }
#pragma omp parallel for schedule(dynamic, 64)
  for (int i = 0; i < m; ++i) {
    float *o = out + (size_t)i * out_dim;
    for (int c = 0; c < out_dim; ++c) o[c] = 0.f;
    for (int j = Ap[i]; j < Ap[i + 1]; ++j) {
      const float *t = tmp + (size_t)Ai[j] * out_dim; float a = Ax[j];
      for (int c = 0; c < out_dim; ++c) o[c] = fmaf(a, t[c], o[c]);
    }
    if (relu) for (int c = 0; c < out_dim; ++c) o[c] = o[c] > 0.f ? o[c] : 0.f;
  }
}

/* ------------------------------------------------------------------ */
/* fp64 cross-checks: D = A * (B * C) with everything accumulated in    */
/* double.  first_is_sparse: B is the CSR (Bp,Bi,Bx) (SpMM-SpMM) else   */
/* B is dense m x kdim and C is kdim x n (GeMM-SpMM, weight [K x N]).   */
/* ------------------------------------------------------------------ */
void orc_chain_f64(int m, int n, const int *Ap, const int *Ai, const float *Ax, int first_is_sparse,
                   const int *Bp, const int *Bi, const float *Bx, int kdim, const float *Bdense,
                   const float *C, double *tmp, double *D) {
#pragma omp parallel for schedule(static)
  for (int i = 0; i < m; ++i) {
    double *t = tmp + (size_t)i * n;
    for (int c = 0; c < n; ++c) t[c] = 0.0;
    if (first_is_sparse) {
      for (int j = Bp[i]; j < Bp[i + 1]; ++j)
        for (int c = 0; c < n; ++c) t[c] += (double)Bx[j] * (double)C[(size_t)Bi[j] * n + c];
    } else {
      for (int k = 0; k < kdim; ++k) {
        double b = Bdense[(size_t)i * kdim + k];
        for (int c = 0; c < n; ++c) t[c] += b * (double)C[(size_t)k * n + c];
      }
    }
  }
#pragma omp parallel for schedule(static)
  for (int i = 0; i < m; ++i) {
    double *o = D + (size_t)i * n;
    for (int c = 0; c < n; ++c) o[c] = 0.0;
    for (int j = Ap[i]; j < Ap[i + 1]; ++j)
      for (int c = 0; c < n; ++c) o[c] += (double)Ax[j] * tmp[(size_t)Ai[j] * n + c];
  }
}

void orc_sddmm_spmm_f64(int m, const int *Ap, const int *Ai, const float *Ax, int kq, int nv,
                        const float *Q, const float *K, const float *V, double *D) {
#pragma omp parallel for schedule(dynamic, 64)
  for (int i = 0; i < m; ++i) {
    double *o = D + (size_t)i * nv;
    for (int c = 0; c < nv; ++c) o[c] = 0.0;
    for (int p = Ap[i]; p < Ap[i + 1]; ++p) {
      double dot = 0.0;
      for (int t = 0; t < kq; ++t) dot += (double)Q[(size_t)i * kq + t] * (double)K[(size_t)Ai[p] * kq + t];
      double s = dot * (double)Ax[p];
      for (int c = 0; c < nv; ++c) o[c] += s * (double)V[(size_t)Ai[p] * nv + c];
    }
  }
}
