/*
 * CPU checker for the convolution path -- TEST INFRASTRUCTURE ONLY.
 *
 * Plain-C restatement of the loop nests the reference uses to lower Conv2D to a GEMM:
 *   im2row / row2im  (NHWC)  pydtnn/cython_modules/im2row_nhwc_cython.pyx:77-97, 174-194
 *   im2col / col2im  (NCHW)  pydtnn/cython_modules/im2col_nchw_cython.pyx:104-124, 224-244
 * and of the index arithmetic they share (row/col numbering, padding test), exported as an
 * integer index map so the map can be compared bit for bit.
 *
 * Nothing in the product path links, loads or calls this file; only the tests, the smoke
 * check and the CPU-baseline leg of the benchmark do.
 */
#include <stdint.h>
#include <string.h>

typedef struct {
    int n, h, w, c;            /* input batch, height, width, channels */
    int kh, kw;                /* filter */
    int vpad, hpad, vstr, hstr, vdil, hdil;
} geom_t;

static inline int out_h(const geom_t *g) { return (g->h + 2 * g->vpad - g->vdil * (g->kh - 1) - 1) / g->vstr + 1; }
static inline int out_w(const geom_t *g) { return (g->w + 2 * g->hpad - g->hdil * (g->kw - 1) - 1) / g->hstr + 1; }

/* ---- index maps (int64 flat offset into x, or -1 for a padding tap) ------------------ */

/* NHWC: map[row, col], row = n*Ho*Wo + xx*Wo + yy, col = cc*kh*kw + ii*kw + jj */
void oracle_index_map_nhwc(const geom_t *g, int64_t *map)
{
    const int hh = out_h(g), ww = out_w(g);
    const int64_t K = (int64_t)g->c * g->kh * g->kw;
#pragma omp parallel for
    for (int nn = 0; nn < g->n; nn++)
        for (int xx = 0; xx < hh; xx++)
            for (int yy = 0; yy < ww; yy++) {
                int64_t row = (int64_t)nn * hh * ww + (int64_t)xx * ww + yy;
                for (int cc = 0; cc < g->c; cc++)
                    for (int ii = 0; ii < g->kh; ii++) {
                        int x_x = g->vstr * xx + g->vdil * ii - g->vpad;
                        for (int jj = 0; jj < g->kw; jj++) {
                            int x_y = g->hstr * yy + g->hdil * jj - g->hpad;
                            int64_t col = (int64_t)cc * g->kh * g->kw + ii * g->kw + jj;
                            int ok = (0 <= x_x && x_x < g->h && 0 <= x_y && x_y < g->w);
                            map[row * K + col] = ok ? (((int64_t)nn * g->h + x_x) * g->w + x_y) * g->c + cc : -1;
                        }
                    }
            }
}

/* NCHW: map[row, col], row = cc*kh*kw + ii*kw + jj, col = n*Ho*Wo + xx*Wo + yy */
void oracle_index_map_nchw(const geom_t *g, int64_t *map)
{
    const int hh = out_h(g), ww = out_w(g);
    const int64_t M = (int64_t)g->n * hh * ww;
#pragma omp parallel for
    for (int cc = 0; cc < g->c; cc++)
        for (int ii = 0; ii < g->kh; ii++)
            for (int jj = 0; jj < g->kw; jj++) {
                int64_t row = (int64_t)cc * g->kh * g->kw + ii * g->kw + jj;
                for (int nn = 0; nn < g->n; nn++)
                    for (int xx = 0; xx < hh; xx++) {
                        int x_x = g->vstr * xx + g->vdil * ii - g->vpad;
                        for (int yy = 0; yy < ww; yy++) {
                            int x_y = g->hstr * yy + g->hdil * jj - g->hpad;
                            int64_t col = (int64_t)nn * hh * ww + (int64_t)xx * ww + yy;
                            int ok = (0 <= x_x && x_x < g->h && 0 <= x_y && x_y < g->w);
                            map[row * M + col] = ok ? (((int64_t)nn * g->c + cc) * g->h + x_x) * g->w + x_y : -1;
                        }
                    }
            }
}

/* ---- gather / scatter-add, generated for float and double ---------------------------- */

#define DEFINE_LOWERING(T, SUF)                                                                   \
void oracle_im2row_nhwc_##SUF(const geom_t *g, const T *x, T *rows)                               \
{                                                                                                 \
    const int hh = out_h(g), ww = out_w(g);                                                       \
    const int64_t K = (int64_t)g->c * g->kh * g->kw;                                              \
    memset(rows, 0, sizeof(T) * (size_t)g->n * hh * ww * K);                                      \
    _Pragma("omp parallel for")                                                                   \
    for (int nn = 0; nn < g->n; nn++)                                                             \
        for (int xx = 0; xx < hh; xx++)                                                           \
            for (int yy = 0; yy < ww; yy++) {                                                     \
                int64_t row = (int64_t)nn * hh * ww + (int64_t)xx * ww + yy;                      \
                for (int cc = 0; cc < g->c; cc++)                                                 \
                    for (int ii = 0; ii < g->kh; ii++) {                                          \
                        int x_x = g->vstr * xx + g->vdil * ii - g->vpad;                          \
                        if (0 <= x_x && x_x < g->h)                                               \
                            for (int jj = 0; jj < g->kw; jj++) {                                  \
                                int x_y = g->hstr * yy + g->hdil * jj - g->hpad;                  \
                                if (0 <= x_y && x_y < g->w) {                                     \
                                    int64_t col = (int64_t)cc * g->kh * g->kw + ii * g->kw + jj;  \
                                    rows[row * K + col] =                                         \
                                        x[(((int64_t)nn * g->h + x_x) * g->w + x_y) * g->c + cc]; \
                                }                                                                 \
                            }                                                                     \
                    }                                                                             \
            }                                                                                     \
}                                                                                                 \
void oracle_row2im_nhwc_##SUF(const geom_t *g, const T *rows, T *x)                               \
{                                                                                                 \
    const int hh = out_h(g), ww = out_w(g);                                                       \
    const int64_t K = (int64_t)g->c * g->kh * g->kw;                                              \
    memset(x, 0, sizeof(T) * (size_t)g->n * g->h * g->w * g->c);                                  \
    _Pragma("omp parallel for")                                                                   \
    for (int nn = 0; nn < g->n; nn++)                                                             \
        for (int xx = 0; xx < hh; xx++)                                                           \
            for (int yy = 0; yy < ww; yy++) {                                                     \
                int64_t row = (int64_t)nn * hh * ww + (int64_t)xx * ww + yy;                      \
                for (int cc = 0; cc < g->c; cc++)                                                 \
                    for (int ii = 0; ii < g->kh; ii++) {                                          \
                        int x_x = g->vstr * xx + g->vdil * ii - g->vpad;                          \
                        if (0 <= x_x && x_x < g->h)                                               \
                            for (int jj = 0; jj < g->kw; jj++) {                                  \
                                int x_y = g->hstr * yy + g->hdil * jj - g->hpad;                  \
                                if (0 <= x_y && x_y < g->w) {                                     \
                                    int64_t col = (int64_t)cc * g->kh * g->kw + ii * g->kw + jj;  \
                                    x[(((int64_t)nn * g->h + x_x) * g->w + x_y) * g->c + cc] +=   \
                                        rows[row * K + col];                                      \
                                }                                                                 \
                            }                                                                     \
                    }                                                                             \
            }                                                                                     \
}                                                                                                 \
void oracle_im2col_nchw_##SUF(const geom_t *g, const T *x, T *cols)                               \
{                                                                                                 \
    const int hh = out_h(g), ww = out_w(g);                                                       \
    const int64_t M = (int64_t)g->n * hh * ww;                                                    \
    memset(cols, 0, sizeof(T) * (size_t)g->c * g->kh * g->kw * M);                                \
    _Pragma("omp parallel for")                                                                   \
    for (int cc = 0; cc < g->c; cc++)                                                             \
        for (int ii = 0; ii < g->kh; ii++)                                                        \
            for (int jj = 0; jj < g->kw; jj++) {                                                  \
                int64_t row = (int64_t)cc * g->kh * g->kw + ii * g->kw + jj;                      \
                for (int nn = 0; nn < g->n; nn++)                                                 \
                    for (int xx = 0; xx < hh; xx++) {                                             \
                        int x_x = g->vstr * xx + g->vdil * ii - g->vpad;                          \
                        if (0 <= x_x && x_x < g->h)                                               \
                            for (int yy = 0; yy < ww; yy++) {                                     \
                                int x_y = g->hstr * yy + g->hdil * jj - g->hpad;                  \
                                if (0 <= x_y && x_y < g->w) {                                     \
                                    int64_t col = (int64_t)nn * hh * ww + (int64_t)xx * ww + yy;  \
                                    cols[row * M + col] =                                         \
                                        x[(((int64_t)nn * g->c + cc) * g->h + x_x) * g->w + x_y]; \
                                }                                                                 \
                            }                                                                     \
                    }                                                                             \
            }                                                                                     \
}                                                                                                 \
void oracle_col2im_nchw_##SUF(const geom_t *g, const T *cols, T *x)                               \
{                                                                                                 \
    const int hh = out_h(g), ww = out_w(g);                                                       \
    const int64_t M = (int64_t)g->n * hh * ww;                                                    \
    memset(x, 0, sizeof(T) * (size_t)g->n * g->c * g->h * g->w);                                  \
    _Pragma("omp parallel for")                                                                   \
    for (int cc = 0; cc < g->c; cc++)                                                             \
        for (int ii = 0; ii < g->kh; ii++)                                                        \
            for (int jj = 0; jj < g->kw; jj++) {                                                  \
                int64_t row = (int64_t)cc * g->kh * g->kw + ii * g->kw + jj;                      \
                for (int nn = 0; nn < g->n; nn++)                                                 \
                    for (int xx = 0; xx < hh; xx++) {                                             \
                        int x_x = g->vstr * xx + g->vdil * ii - g->vpad;                          \
                        if (0 <= x_x && x_x < g->h)                                               \
                            for (int yy = 0; yy < ww; yy++) {                                     \
                                int x_y = g->hstr * yy + g->hdil * jj - g->hpad;                  \
                                if (0 <= x_y && x_y < g->w) {                                     \
                                    int64_t col = (int64_t)nn * hh * ww + (int64_t)xx * ww + yy;  \
                                    x[(((int64_t)nn * g->c + cc) * g->h + x_x) * g->w + x_y] +=   \
                                        cols[row * M + col];                                      \
                                }                                                                 \
                            }                                                                     \
                    }                                                                             \
            }                                                                                     \
}

DEFINE_LOWERING(float, f32)
DEFINE_LOWERING(double, f64)
