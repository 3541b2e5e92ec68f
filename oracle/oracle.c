/*
 * CPU oracle (plain C): see oracle.h for what each function restates and how parity of this
 * file is pinned. TEST INFRASTRUCTURE ONLY: never linked into or called from product code.
 *
 * Structure shared by the element-wise kernels, mirroring the reference's emitted drivers
 * (src/backend/stitch_and_generate_cpu.cpp:103-215): split the merged work among threads,
 * count each thread's outputs, take a serial exclusive prefix, then fill. The reference cuts
 * work between arbitrary elements; this restatement cuts CSR work between rows (COO3 work
 * between elements). The results are the canonical sorted union / intersection either way,
 * so the outputs are identical for any thread count.
 */
#define _GNU_SOURCE
#include "oracle.h"

#include <pthread.h>
#include <stdlib.h>
#include <string.h>

/* ------------------------------------------------------------------ thread helper ---- */

typedef void (*block_fn)(void *ctx, int tid, int nthreads);

typedef struct {
    block_fn fn;
    void *ctx;
    int tid, nthreads;
} block_arg;

static void *block_entry(void *p) {
    block_arg *a = (block_arg *)p;
    a->fn(a->ctx, a->tid, a->nthreads);
    return NULL;
}

static void run_blocks(int nthreads, block_fn fn, void *ctx) {
    if (nthreads <= 1) {
        fn(ctx, 0, 1);
        return;
    }
    pthread_t *th = (pthread_t *)malloc(sizeof(pthread_t) * (size_t)nthreads);
    block_arg *args = (block_arg *)malloc(sizeof(block_arg) * (size_t)nthreads);
    for (int t = 0; t < nthreads; ++t) {
        args[t].fn = fn;
        args[t].ctx = ctx;
        args[t].tid = t;
        args[t].nthreads = nthreads;
        if (t > 0) pthread_create(&th[t], NULL, block_entry, &args[t]);
    }
    block_entry(&args[0]);
    for (int t = 1; t < nthreads; ++t) pthread_join(th[t], NULL);
    free(th);
    free(args);
}

static int clamp_threads(int nthreads) { return nthreads < 1 ? 1 : (nthreads > 1024 ? 1024 : nthreads); }

/* ------------------------------------------------------------ CSR add / mul / add3 ---- */

enum { MODE_UNION = 0, MODE_INTERSECT = 1 };

typedef struct {
    int nops, mode;
    int32_t rows;
    const int32_t *rp[3];
    const int32_t *col[3];
    const float *val[3];
    int32_t *z_rp;
    int32_t *z_col;
    float *z_val;
    int32_t *row_cut; /* nthreads + 1 row boundaries */
    int fill;
} csr_ctx;

/* Work (stored entries of all operands) in rows [0, i): the quantity the reference bisects
 * on to find a thread's first row (src/backend/tensor.cpp:163-445 work functions,
 * src/backend/partition.cpp:628-811). */
static int64_t csr_work_before(const csr_ctx *c, int32_t i) {
    int64_t w = 0;
    for (int o = 0; o < c->nops; ++o) w += (int64_t)c->rp[o][i] - c->rp[o][0];
    return w;
}

static int32_t csr_row_for_work(const csr_ctx *c, int64_t target) {
    int32_t lo = 0, hi = c->rows; /* first row whose preceding work >= target */
    while (lo < hi) {
        int32_t mid = lo + (hi - lo) / 2;
        if (csr_work_before(c, mid) < target) lo = mid + 1; else hi = mid;
    }
    return lo;
}

/* One row: sorted k-way merge. With out == 0 only counts. Returns outputs of the row. */
static int32_t csr_merge_row(const csr_ctx *c, int32_t i, int32_t out_base, int write) {
    int32_t p[3], e[3];
    for (int o = 0; o < c->nops; ++o) {
        p[o] = c->rp[o][i];
        e[o] = c->rp[o][i + 1];
    }
    int32_t n = 0;
    for (;;) {
        int any = 0, all = 1;
        int32_t m = 0;
        for (int o = 0; o < c->nops; ++o) {
            if (p[o] < e[o]) {
                int32_t v = c->col[o][p[o]];
                if (!any || v < m) m = v;
                any = 1;
            } else {
                all = 0;
            }
        }
        if (!any) break;
        if (c->mode == MODE_INTERSECT && !all) break;
        int hits = 0;
        float acc = 0.0f;
        for (int o = 0; o < c->nops; ++o) {
            if (p[o] < e[o] && c->col[o][p[o]] == m) {
                float v = c->val[o][p[o]];
                if (c->mode == MODE_INTERSECT) acc = hits ? acc * v : v;
                else acc = hits ? acc + v : v; /* left-to-right: (a + b) + c */
                ++hits;
                ++p[o];
            }
        }
        if (c->mode == MODE_INTERSECT && hits != c->nops) continue;
        if (write) {
            c->z_col[out_base + n] = m;
            c->z_val[out_base + n] = acc;
        }
        ++n;
    }
    return n;
}

static void csr_block(void *ctx, int tid, int nthreads) {
    (void)nthreads;
    csr_ctx *c = (csr_ctx *)ctx;
    for (int32_t i = c->row_cut[tid]; i < c->row_cut[tid + 1]; ++i) {
        if (!c->fill) c->z_rp[i + 1] = csr_merge_row(c, i, 0, 0);
        else csr_merge_row(c, i, c->z_rp[i], 1);
    }
}

static int64_t csr_merge(csr_ctx *c, int nthreads) {
    if (c->rows < 0) return -1;
    nthreads = clamp_threads(nthreads);
    c->row_cut = (int32_t *)malloc(sizeof(int32_t) * (size_t)(nthreads + 1));
    int64_t total = csr_work_before(c, c->rows);
    int64_t per_thread = total / nthreads + 1; /* src/backend/stitch_and_generate.cpp:106-111 */
    c->row_cut[0] = 0;
    for (int t = 1; t < nthreads; ++t) c->row_cut[t] = csr_row_for_work(c, (int64_t)t * per_thread);
    c->row_cut[nthreads] = c->rows;
    for (int t = 1; t <= nthreads; ++t)
        if (c->row_cut[t] < c->row_cut[t - 1]) c->row_cut[t] = c->row_cut[t - 1];

    c->z_rp[0] = 0;
    c->fill = 0;
    run_blocks(nthreads, csr_block, c);
    int64_t run = 0; /* serial prefix, src/backend/stitch_and_generate_cpu.cpp:156-215 */
    for (int32_t i = 0; i < c->rows; ++i) {
        run += c->z_rp[i + 1];
        c->z_rp[i + 1] = (int32_t)run;
    }
    c->fill = 1;
    run_blocks(nthreads, csr_block, c);
    free(c->row_cut);
    return run;
}

int64_t orc_csr_add(int32_t rows, const int32_t *a_row_ptr, const int32_t *a_col,
                    const float *a_val, const int32_t *b_row_ptr, const int32_t *b_col,
                    const float *b_val, int32_t *z_row_ptr, int32_t *z_col, float *z_val,
                    int nthreads) {
    csr_ctx c = {2, MODE_UNION, rows, {a_row_ptr, b_row_ptr, NULL}, {a_col, b_col, NULL},
                 {a_val, b_val, NULL}, z_row_ptr, z_col, z_val, NULL, 0};
    return csr_merge(&c, nthreads);
}

int64_t orc_csr_mul(int32_t rows, const int32_t *a_row_ptr, const int32_t *a_col,
                    const float *a_val, const int32_t *b_row_ptr, const int32_t *b_col,
                    const float *b_val, int32_t *z_row_ptr, int32_t *z_col, float *z_val,
                    int nthreads) {
    csr_ctx c = {2, MODE_INTERSECT, rows, {a_row_ptr, b_row_ptr, NULL}, {a_col, b_col, NULL},
                 {a_val, b_val, NULL}, z_row_ptr, z_col, z_val, NULL, 0};
    return csr_merge(&c, nthreads);
}

int64_t orc_csr_add3(int32_t rows, const int32_t *a_row_ptr, const int32_t *a_col,
                     const float *a_val, const int32_t *b_row_ptr, const int32_t *b_col,
                     const float *b_val, const int32_t *c_row_ptr, const int32_t *c_col,
                     const float *c_val, int32_t *z_row_ptr, int32_t *z_col, float *z_val,
                     int nthreads) {
    csr_ctx c = {3, MODE_UNION, rows, {a_row_ptr, b_row_ptr, c_row_ptr}, {a_col, b_col, c_col},
                 {a_val, b_val, c_val}, z_row_ptr, z_col, z_val, NULL, 0};
    return csr_merge(&c, nthreads);
}

/* ----------------------------------------------------------------------- COO3 add ---- */

typedef struct {
    int32_t na, nb;
    const int32_t *ai, *aj, *ak, *bi, *bj, *bk;
    const float *av, *bv;
    int32_t *zi, *zj, *zk;
    float *zv;
    int32_t *cut_a, *cut_b; /* nthreads + 1 */
    int64_t *count;         /* nthreads + 1, exclusive prefix after the count phase */
    int fill;
} coo3_ctx;

/* Lexicographic compare of A[x] with B[y]: <0, 0, >0 (tuple compare,
 * src/backend/tensor.cpp:447-560). */
static int coo3_cmp(const coo3_ctx *c, int32_t x, int32_t y) {
    if (c->ai[x] != c->bi[y]) return c->ai[x] < c->bi[y] ? -1 : 1;
    if (c->aj[x] != c->bj[y]) return c->aj[x] < c->bj[y] ? -1 : 1;
    if (c->ak[x] != c->bk[y]) return c->ak[x] < c->bk[y] ? -1 : 1;
    return 0;
}

/* Merge-path split of diagonal d, equal coordinates ordered A first; an equal pair is never
 * separated (src/backend/partition.cpp:813-993, tie rule :964-983). */
static void coo3_split(const coo3_ctx *c, int64_t d, int32_t *x_out, int32_t *y_out) {
    int64_t lo = d - c->nb > 0 ? d - c->nb : 0;
    int64_t hi = d < c->na ? d : c->na;
    while (lo < hi) {
        int64_t mid = lo + (hi - lo) / 2;
        if (coo3_cmp(c, (int32_t)mid, (int32_t)(d - 1 - mid)) <= 0) lo = mid + 1; else hi = mid;
    }
    int32_t x = (int32_t)lo, y = (int32_t)(d - lo);
    if (x > 0 && y < c->nb && coo3_cmp(c, x - 1, y) == 0) ++y;
    *x_out = x;
    *y_out = y;
}

static void coo3_block(void *ctx, int tid, int nthreads) {
    (void)nthreads;
    coo3_ctx *c = (coo3_ctx *)ctx;
    int32_t x = c->cut_a[tid], xe = c->cut_a[tid + 1];
    int32_t y = c->cut_b[tid], ye = c->cut_b[tid + 1];
    int64_t o = c->fill ? c->count[tid] : 0, o0 = o;
    while (x < xe || y < ye) {
        int cmp = (x < xe && y < ye) ? coo3_cmp(c, x, y) : (x < xe ? -1 : 1);
        if (c->fill) {
            if (cmp <= 0) {
                c->zi[o] = c->ai[x]; c->zj[o] = c->aj[x]; c->zk[o] = c->ak[x];
                c->zv[o] = cmp == 0 ? c->av[x] + c->bv[y] : c->av[x];
            } else {
                c->zi[o] = c->bi[y]; c->zj[o] = c->bj[y]; c->zk[o] = c->bk[y];
                c->zv[o] = c->bv[y];
            }
        }
        if (cmp <= 0) ++x;
        if (cmp >= 0) ++y;
        ++o;
    }
    if (!c->fill) c->count[tid] = o - o0;
}

int64_t orc_coo3_add(int32_t na, const int32_t *ai, const int32_t *aj, const int32_t *ak,
                     const float *av, int32_t nb, const int32_t *bi, const int32_t *bj,
                     const int32_t *bk, const float *bv, int32_t *zi, int32_t *zj, int32_t *zk,
                     float *zv, int nthreads) {
    if (na < 0 || nb < 0) return -1;
    nthreads = clamp_threads(nthreads);
    coo3_ctx c = {na, nb, ai, aj, ak, bi, bj, bk, av, bv, zi, zj, zk, zv, NULL, NULL, NULL, 0};
    c.cut_a = (int32_t *)malloc(sizeof(int32_t) * (size_t)(nthreads + 1));
    c.cut_b = (int32_t *)malloc(sizeof(int32_t) * (size_t)(nthreads + 1));
    c.count = (int64_t *)calloc((size_t)(nthreads + 1), sizeof(int64_t));
    int64_t total = (int64_t)na + nb;
    int64_t per_thread = total / nthreads + 1;
    for (int t = 0; t <= nthreads; ++t) {
        int64_t d = (int64_t)t * per_thread;
        if (t == nthreads || d >= total) {
            c.cut_a[t] = na;
            c.cut_b[t] = nb;
        } else {
            coo3_split(&c, d, &c.cut_a[t], &c.cut_b[t]);
        }
    }
    run_blocks(nthreads, coo3_block, &c);
    int64_t run = 0;
    for (int t = 0; t <= nthreads; ++t) {
        int64_t n = c.count[t];
        c.count[t] = run;
        run += n;
    }
    c.fill = 1;
    run_blocks(nthreads, coo3_block, &c);
    free(c.cut_a);
    free(c.cut_b);
    free(c.count);
    return run;
}

/* ----------------------------------------------------------------------- CSF3 add ---- */

int64_t orc_csf3_add(int32_t na_i, const int32_t *a_i_idx, const int32_t *a_j_ptr,
                     const int32_t *a_j_idx, const int32_t *a_k_ptr, const int32_t *a_k_idx,
                     const float *a_val, int32_t nb_i, const int32_t *b_i_idx,
                     const int32_t *b_j_ptr, const int32_t *b_j_idx, const int32_t *b_k_ptr,
                     const int32_t *b_k_idx, const float *b_val, int32_t *z_i_idx,
                     int32_t *z_j_ptr, int32_t *z_j_idx, int32_t *z_k_ptr, int32_t *z_k_idx,
                     float *z_val, int32_t *counts) {
    if (na_i < 0 || nb_i < 0) return -1;
    int32_t zi = 0, zj = 0, zk = 0;
    int32_t pa = 0, pb = 0;
    z_j_ptr[0] = 0;
    z_k_ptr[0] = 0;
    while (pa < na_i || pb < nb_i) {
        int has_a = pa < na_i, has_b = pb < nb_i;
        int take_a = has_a && (!has_b || a_i_idx[pa] <= b_i_idx[pb]);
        int take_b = has_b && (!has_a || b_i_idx[pb] <= a_i_idx[pa]);
        z_i_idx[zi] = take_a ? a_i_idx[pa] : b_i_idx[pb];
        int32_t ja = take_a ? a_j_ptr[pa] : 0, ja_end = take_a ? a_j_ptr[pa + 1] : 0;
        int32_t jb = take_b ? b_j_ptr[pb] : 0, jb_end = take_b ? b_j_ptr[pb + 1] : 0;
        while (ja < ja_end || jb < jb_end) {
            int hja = ja < ja_end, hjb = jb < jb_end;
            int tja = hja && (!hjb || a_j_idx[ja] <= b_j_idx[jb]);
            int tjb = hjb && (!hja || b_j_idx[jb] <= a_j_idx[ja]);
            z_j_idx[zj] = tja ? a_j_idx[ja] : b_j_idx[jb];
            int32_t ka = tja ? a_k_ptr[ja] : 0, ka_end = tja ? a_k_ptr[ja + 1] : 0;
            int32_t kb = tjb ? b_k_ptr[jb] : 0, kb_end = tjb ? b_k_ptr[jb + 1] : 0;
            while (ka < ka_end || kb < kb_end) {
                int hka = ka < ka_end, hkb = kb < kb_end;
                int tka = hka && (!hkb || a_k_idx[ka] <= b_k_idx[kb]);
                int tkb = hkb && (!hka || b_k_idx[kb] <= a_k_idx[ka]);
                z_k_idx[zk] = tka ? a_k_idx[ka] : b_k_idx[kb];
                z_val[zk] = (tka && tkb) ? a_val[ka] + b_val[kb] : (tka ? a_val[ka] : b_val[kb]);
                ++zk;
                ka += tka;
                kb += tkb;
            }
            ++zj;
            z_k_ptr[zj] = zk;
            ja += tja;
            jb += tjb;
        }
        ++zi;
        z_j_ptr[zi] = zj;
        pa += take_a;
        pb += take_b;
    }
    if (counts) {
        counts[0] = zi;
        counts[1] = zj;
        counts[2] = zk;
    }
    return zk;
}

/* ------------------------------------------------------------------------- SpGEMM ---- */

typedef struct {
    int32_t k;
    float pf;
    double pd;
} esc_item;

typedef struct {
    int32_t rows, b_cols;
    const int32_t *a_rp, *a_col, *b_rp, *b_col;
    const float *a_val, *b_val;
    int32_t *c_rp;
    int32_t *c_col;
    float *c_val;
    double *c_val64, *c_abs64;
    int64_t *products; /* per thread */
    int numeric;
} esc_ctx;

static void esc_rows_of(const esc_ctx *c, int tid, int nthreads, int32_t *r0, int32_t *r1) {
    int64_t per = ((int64_t)c->rows + nthreads - 1) / nthreads;
    int64_t a = per * tid, b = a + per;
    *r0 = (int32_t)(a > c->rows ? c->rows : a);
    *r1 = (int32_t)(b > c->rows ? c->rows : b);
}

/* Stable bottom-up merge sort by key k; ties keep expansion order (ascending j). */
static esc_item *esc_sort(esc_item *buf, esc_item *tmp, int64_t n) {
    esc_item *src = buf, *dst = tmp;
    for (int64_t w = 1; w < n; w *= 2) {
        for (int64_t lo = 0; lo < n; lo += 2 * w) {
            int64_t mid = lo + w < n ? lo + w : n, hi = lo + 2 * w < n ? lo + 2 * w : n;
            int64_t x = lo, y = mid, o = lo;
            while (x < mid && y < hi) dst[o++] = (src[y].k < src[x].k) ? src[y++] : src[x++];
            while (x < mid) dst[o++] = src[x++];
            while (y < hi) dst[o++] = src[y++];
        }
        esc_item *t = src; src = dst; dst = t;
    }
    return src;
}

static void esc_block(void *ctx, int tid, int nthreads) {
    esc_ctx *c = (esc_ctx *)ctx;
    int32_t r0, r1;
    esc_rows_of(c, tid, nthreads, &r0, &r1);
    int64_t max_p = 0, sum_p = 0;
    for (int32_t i = r0; i < r1; ++i) {
        int64_t p = 0;
        for (int32_t q = c->a_rp[i]; q < c->a_rp[i + 1]; ++q) {
            int32_t j = c->a_col[q];
            p += c->b_rp[j + 1] - c->b_rp[j]; /* expand phase 1, compute.cpp:541-611 */
        }
        sum_p += p;
        if (p > max_p) max_p = p;
    }
    if (!c->numeric) c->products[tid] = sum_p;
    esc_item *buf = (esc_item *)malloc(sizeof(esc_item) * (size_t)(max_p + 1));
    esc_item *tmp = (esc_item *)malloc(sizeof(esc_item) * (size_t)(max_p + 1));
    for (int32_t i = r0; i < r1; ++i) {
        int64_t n = 0;
        for (int32_t q = c->a_rp[i]; q < c->a_rp[i + 1]; ++q) { /* expand phase 2 */
            int32_t j = c->a_col[q];
            for (int32_t s = c->b_rp[j]; s < c->b_rp[j + 1]; ++s) {
                buf[n].k = c->b_col[s];
                if (c->numeric) {
                    buf[n].pf = c->a_val[q] * c->b_val[s];
                    buf[n].pd = (double)c->a_val[q] * (double)c->b_val[s];
                }
                ++n;
            }
        }
        esc_item *s = esc_sort(buf, tmp, n); /* sort */
        int32_t out = c->numeric ? c->c_rp[i] : 0;
        int32_t uniq = 0;
        for (int64_t x = 0; x < n;) { /* compress: sum runs of equal k */
            int64_t y = x;
            float accf = 0.0f;
            double accd = 0.0, acca = 0.0;
            while (y < n && s[y].k == s[x].k) {
                if (c->numeric) {
                    accf = (y == x) ? s[y].pf : accf + s[y].pf;
                    accd += s[y].pd;
                    acca += s[y].pd < 0 ? -s[y].pd : s[y].pd;
                }
                ++y;
            }
            if (c->numeric) {
                c->c_col[out + uniq] = s[x].k;
                c->c_val[out + uniq] = accf;
                if (c->c_val64) c->c_val64[out + uniq] = accd;
                if (c->c_abs64) c->c_abs64[out + uniq] = acca;
            }
            ++uniq;
            x = y;
        }
        if (!c->numeric) c->c_rp[i + 1] = uniq;
    }
    free(buf);
    free(tmp);
}

int64_t orc_spgemm_symbolic(int32_t rows, int32_t b_cols, const int32_t *a_row_ptr,
                            const int32_t *a_col, const int32_t *b_row_ptr,
                            const int32_t *b_col, int32_t *c_row_ptr, int64_t *products,
                            int nthreads) {
    if (rows < 0) return -1;
    nthreads = clamp_threads(nthreads);
    esc_ctx c = {rows, b_cols, a_row_ptr, a_col, b_row_ptr, b_col, NULL, NULL, c_row_ptr,
                 NULL, NULL, NULL, NULL, NULL, 0};
    c.products = (int64_t *)calloc((size_t)nthreads, sizeof(int64_t));
    c_row_ptr[0] = 0;
    run_blocks(nthreads, esc_block, &c);
    int64_t run = 0, p = 0;
    for (int32_t i = 0; i < rows; ++i) {
        run += c_row_ptr[i + 1];
        c_row_ptr[i + 1] = (int32_t)run;
    }
    for (int t = 0; t < nthreads; ++t) p += c.products[t];
    if (products) *products = p;
    free(c.products);
    return run;
}

int64_t orc_spgemm_numeric(int32_t rows, int32_t b_cols, const int32_t *a_row_ptr,
                           const int32_t *a_col, const float *a_val, const int32_t *b_row_ptr,
                           const int32_t *b_col, const float *b_val, const int32_t *c_row_ptr,
                           int32_t *c_col, float *c_val, double *c_val64, double *c_abs64,
                           int nthreads) {
    if (rows < 0) return -1;
    nthreads = clamp_threads(nthreads);
    esc_ctx c = {rows, b_cols, a_row_ptr, a_col, b_row_ptr, b_col, a_val, b_val,
                 (int32_t *)c_row_ptr, c_col, c_val, c_val64, c_abs64, NULL, 1};
    run_blocks(nthreads, esc_block, &c);
    return c_row_ptr[rows];
}
