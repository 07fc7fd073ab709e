// Sparse handling of the fp32 accumulation image of the backward pass.
//
// With a 16-bit value dtype the backward scatters into an fp32 image of grad_value that is zero-filled
// before and converted afterwards.  Both are dense passes over the image (4 + 4 + 2 bytes per element),
// whatever the number of sampling points.  When the points touch only a part of the image -- a few hundred
// object queries looking into a large volume, reference call site ops3d/flash_deform_attn.py:121-133 with
// num_query << num_value -- the dense passes dominate the step.  The two kernels here walk the POINT list
// instead and visit exactly the rows the scatter can touch (the 8 corner cells of every point, one head
// row of D channels each):
//
//   kCast = false   before the scatter: write zeros to those rows of the image;
//   kCast = true    after the scatter:  convert those rows into grad_value (which the host zero-filled).
//
// Rows that several points share are visited once per point; every visitor writes the same bytes, so no
// ordering between them is needed.  The rest of the image is never read or written and may hold anything.
// The corner cells and their validity come from point_geometry(), the routine the scatter kernels use, so
// the three passes agree on the set of rows bit for bit.
#pragma once

#include "fda_device.cuh"

namespace fda {

// One thread per (point, 4-channel vector of the row); `vecs` = D / 4 threads cover a row.
template <typename VT, typename PT, bool kCast>
__global__ void __launch_bounds__(256) fda_touch_rows_kernel(const Problem p, VT *__restrict__ grad_value,
                                                             unsigned long long total_threads, int vecs) {
    const unsigned long long t = (unsigned long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= total_threads) return;
    const unsigned long long point = t / (unsigned)vecs;
    const int vec = (int)(t - point * (unsigned)vecs);
    const unsigned long long row = point / (unsigned)p.LK;  // b * Q * G + q * G + g
    const int i = (int)(point - row * (unsigned)p.LK);      // point of the row; its level is i / K
    const int b = (int)(row / (unsigned)p.rows_per_b);
    const int g = (int)(row % (unsigned)p.G);
    // Every thread reads its level's extents itself, side by side with the point's coordinates: one memory latency,
    // where a level table built by one thread per block and a barrier cost more than the rest of this short kernel.
    const int l = i >> (2 + p.k_shift);
    const PT *c = static_cast<const PT *>(p.packed) + row * (unsigned long long)(4 * p.LK) + 3 * i;
    const float x = load1<PT>(c), y = load1<PT>(c + 1), z = load1<PT>(c + 2);
    LevelGeom lv;
    lv.D = (int)p.shapes[3 * l];
    lv.H = (int)p.shapes[3 * l + 1];
    lv.W = (int)p.shapes[3 * l + 2];
    lv.start = (int)p.lsi[l];
    lv.keep = 0;
    lv.fD = (float)lv.D; lv.fH = (float)lv.H; lv.fW = (float)lv.W;
    PointGeom pg;
    point_geometry(lv, p.GD, x, y, z, pg);

    const size_t base = ((size_t)b * p.N + lv.start) * (size_t)p.GD + (size_t)g * p.D + (size_t)vec * 4;
    float *image = p.accum + base;
#pragma unroll
    for (int n = 0; n < 8; ++n) {
        if (!(pg.zin[n >> 2] && pg.yin[(n >> 1) & 1] && pg.xin[n & 1])) continue;
        if (kCast) {
            const float4 f = *reinterpret_cast<const float4 *>(image + pg.off[n]);
            store4<VT>(grad_value + base + pg.off[n], f);
        } else {
            *reinterpret_cast<float4 *>(image + pg.off[n]) = make_float4(0.f, 0.f, 0.f, 0.f);
        }
    }
}

}  // namespace fda
