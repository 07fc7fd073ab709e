/*
 * Plain-C restatement of Flash Deformable 3D Attention (forward and analytic
 * backward).  TEST INFRASTRUCTURE ONLY: it is the checker for the CUDA kernels
 * and is never linked into, imported by, or called from the product library.
 *
 * What it follows in the reference (paths inside cell-observatory/ops3d):
 *   forward   csrc/cuda/flash_deform_im2col_cuda.cuh:216-281  (softmax over the
 *             L*K logits of one (b,q,g); per point x_im = loc*size - 0.5)
 *             csrc/cuda/common.h:52-138  (8-corner trilinear gather, each
 *             corner zero when outside the level)
 *   backward  csrc/cuda/common.h:141-354 (grad_value scatter w*alpha*g,
 *             d/dx,dy,dz scaled by size*alpha, d/dalpha = <sample, g>)
 *             csrc/cuda/flash_deform_col2im_cuda.cuh:413-427 (softmax Jacobian)
 *   semantics ops3d/flash_deform_attn.py:139-165 (grid_sample, bilinear,
 *             padding zeros, align_corners=False) -- the parity target.
 *
 * Layouts (all contiguous):
 *   value   [B][N][G][D]           N = sum_l Dl*Hl*Wl, level-major, (z,y,x) row-major
 *   shapes  [L][3] = (Dl,Hl,Wl)    lsi [L] = first cell of each level
 *   packed  [B][Q][G][L*K*4]       planar: L*K*3 coords (x,y,z per point) then L*K logits
 *   out     [B][Q][G][D]
 * Inputs are fp32; accumulation is in double so that this restatement is the
 * more exact side of every comparison.
 *
 * Coordinates are un-normalised with grid_sample's own fp32 sequence
 * g = 2*loc - 1;  c = ((g + 1) * size - 1) / 2   so that corner indices and
 * weights agree with the PyTorch oracle even next to cell boundaries.
 *
 * Parity pin: checked against tests/golden/ fixtures, which were produced by
 * the reference package itself (tests/golden/make_golden.py).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define FDA_MAX_POINTS 1024

static inline float unnormalize(float loc, int size) {
    volatile float g = 2.0f * loc - 1.0f; /* volatile: keep the fp32 roundings separate */
    volatile float t = g + 1.0f;
    volatile float u = t * (float)size;
    volatile float v = u - 1.0f;
    return v / 2.0f;
}

typedef struct {
    int inside[8];
    int64_t cell[8];
    double w[8];       /* trilinear weight */
    double dwx[8];     /* d w / d x_im */
    double dwy[8];
    double dwz[8];
} corners_t;

static void corners_of(float loc_x, float loc_y, float loc_z, int Dl, int Hl, int Wl, corners_t *c) {
    const float xi = unnormalize(loc_x, Wl);
    const float yi = unnormalize(loc_y, Hl);
    const float zi = unnormalize(loc_z, Dl);
    const float xf = floorf(xi), yf = floorf(yi), zf = floorf(zi);
    /* weights as grid_sample forms them: (x0+1) - x and x - x0 */
    const double wx[2] = {(double)((xf + 1.0f) - xi), (double)(xi - xf)};
    const double wy[2] = {(double)((yf + 1.0f) - yi), (double)(yi - yf)};
    const double wz[2] = {(double)((zf + 1.0f) - zi), (double)(zi - zf)};
    const double sgn[2] = {-1.0, 1.0};
    int n = 0;
    for (int dz = 0; dz < 2; ++dz)
        for (int dy = 0; dy < 2; ++dy)
            for (int dx = 0; dx < 2; ++dx, ++n) {
                /* compare in floating point first: huge or non-finite coordinates never index */
                const float cx = xf + (float)dx, cy = yf + (float)dy, cz = zf + (float)dz;
                const int in = (cx >= 0.0f && cx < (float)Wl && cy >= 0.0f && cy < (float)Hl &&
                                cz >= 0.0f && cz < (float)Dl);
                c->inside[n] = in;
                c->cell[n] = in ? (((int64_t)cz * Hl + (int64_t)cy) * Wl + (int64_t)cx) : 0;
                c->w[n] = wz[dz] * wy[dy] * wx[dx];
                c->dwx[n] = sgn[dx] * wy[dy] * wz[dz];
                c->dwy[n] = sgn[dy] * wx[dx] * wz[dz];
                c->dwz[n] = sgn[dz] * wx[dx] * wy[dy];
            }
}

static void softmax_row(const float *logits, int n, double *p) {
    float m = logits[0];
    for (int i = 1; i < n; ++i) m = logits[i] > m ? logits[i] : m;
    double s = 0.0;
    for (int i = 0; i < n; ++i) { p[i] = exp((double)logits[i] - (double)m); s += p[i]; }
    for (int i = 0; i < n; ++i) p[i] /= s;
}

int fda_oracle_forward(const float *value, const int64_t *shapes, const int64_t *lsi,
                       const float *packed, int B, int N, int G, int D, int L, int K, int Q,
                       float *out) {
    const int LK = L * K;
    if (LK > FDA_MAX_POINTS || LK <= 0) return 1;
    const int64_t rows = (int64_t)B * Q;

    for (int64_t r = 0; r < rows; ++r) {
        const int b = (int)(r / Q);
        double p[FDA_MAX_POINTS];
        double *acc = (double *)malloc(sizeof(double) * (size_t)D);
        corners_t c;
        for (int g = 0; g < G; ++g) {
            const float *row = packed + ((int64_t)r * G + g) * LK * 4;
            softmax_row(row + 3 * LK, LK, p);
            for (int d = 0; d < D; ++d) acc[d] = 0.0;
            for (int i = 0; i < LK; ++i) {
                const int l = i / K;
                const int Dl = (int)shapes[3 * l], Hl = (int)shapes[3 * l + 1], Wl = (int)shapes[3 * l + 2];
                corners_of(row[3 * i], row[3 * i + 1], row[3 * i + 2], Dl, Hl, Wl, &c);
                for (int n = 0; n < 8; ++n) {
                    if (!c.inside[n]) continue;
                    const float *v = value + (((int64_t)b * N + lsi[l] + c.cell[n]) * G + g) * D;
                    const double w = p[i] * c.w[n];
                    for (int d = 0; d < D; ++d) acc[d] += w * (double)v[d];
                }
            }
            float *o = out + ((int64_t)r * G + g) * D;
            for (int d = 0; d < D; ++d) o[d] = (float)acc[d];
        }
        free(acc);
    }
    return 0;
}

/* grad_value [B][N][G][D] and grad_packed [B][Q][G][L*K*4] (same planar layout as
 * packed: coordinate gradients, then gradients w.r.t. the raw logits).  The loop
 * runs over (b,g) pairs; each pair owns a disjoint slice of grad_value, which is
 * accumulated in double and rounded to fp32 once.  Single-threaded by design
 * (this is a checker for small cases). */
int fda_oracle_backward(const float *value, const int64_t *shapes, const int64_t *lsi,
                        const float *packed, const float *grad_out, int B, int N, int G, int D,
                        int L, int K, int Q, float *grad_value, float *grad_packed) {
    const int LK = L * K;
    if (LK > FDA_MAX_POINTS || LK <= 0) return 1;
    int status = 0;

    for (int bg = 0; bg < B * G; ++bg) {
        const int b = bg / G, g = bg % G;
        double *gv = (double *)calloc((size_t)N * D, sizeof(double));
        if (!gv) { status = 2; continue; }
        double p[FDA_MAX_POINTS], dalpha[FDA_MAX_POINTS];
        corners_t c;
        for (int q = 0; q < Q; ++q) {
            const int64_t rg = ((int64_t)b * Q + q) * G + g;
            const float *row = packed + rg * LK * 4;
            float *grow = grad_packed + rg * LK * 4;
            const float *go = grad_out + rg * D;
            softmax_row(row + 3 * LK, LK, p);
            for (int i = 0; i < LK; ++i) {
                const int l = i / K;
                const int Dl = (int)shapes[3 * l], Hl = (int)shapes[3 * l + 1], Wl = (int)shapes[3 * l + 2];
                corners_of(row[3 * i], row[3 * i + 1], row[3 * i + 2], Dl, Hl, Wl, &c);
                double gx = 0.0, gy = 0.0, gz = 0.0, da = 0.0;
                for (int n = 0; n < 8; ++n) {
                    if (!c.inside[n]) continue;
                    const int64_t cell = lsi[l] + c.cell[n];
                    const float *v = value + (((int64_t)b * N + cell) * G + g) * D;
                    double *acc = gv + cell * D;
                    double dot = 0.0;
                    const double w = p[i] * c.w[n];
                    for (int d = 0; d < D; ++d) {
                        dot += (double)v[d] * (double)go[d];
                        acc[d] += w * (double)go[d];
                    }
                    da += c.w[n] * dot;
                    gx += c.dwx[n] * dot;
                    gy += c.dwy[n] * dot;
                    gz += c.dwz[n] * dot;
                }
                grow[3 * i + 0] = (float)(p[i] * (double)Wl * gx);
                grow[3 * i + 1] = (float)(p[i] * (double)Hl * gy);
                grow[3 * i + 2] = (float)(p[i] * (double)Dl * gz);
                dalpha[i] = da;
            }
            double s = 0.0;
            for (int i = 0; i < LK; ++i) s += p[i] * dalpha[i];
            for (int i = 0; i < LK; ++i) grow[3 * LK + i] = (float)(p[i] * (dalpha[i] - s));
        }
        for (int64_t n = 0; n < N; ++n) {
            float *dst = grad_value + (((int64_t)b * N + n) * G + g) * D;
            const double *src = gv + n * D;
            for (int d = 0; d < D; ++d) dst[d] = (float)src[d];
        }
        free(gv);
    }
    return status;
}
