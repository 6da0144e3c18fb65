// 3-nearest-neighbour search over a uniform cell grid, shared by the sm_100a kernel and the CPU twin.
//
// Stands in for `distCUDA2` of the simple-knn submodule, which the reference imports
// (scene/gaussian_nn_module.py:413-414) but does not ship: mean of the squared distances to the three nearest
// other points. Points are sorted by cell; a query visits the cells within Chebyshev radius r = 1, 2, ... of its
// own cell and stops as soon as its third-best distance cannot be beaten by any unvisited cell (exact search).
#pragma once
#include "rgs_math.h"

struct RgsKnnGrid {
    float lo[3];
    float cell;
    int dims[3];
};

RGS_HD void rgs_knn_insert(float d, float* best) {
    if (d < best[2]) {
        if (d < best[1]) {
            best[2] = best[1];
            if (d < best[0]) { best[1] = best[0]; best[0] = d; } else { best[1] = d; }
        } else {
            best[2] = d;
        }
    }
}

// pts: points sorted by cell id; cell_start: (ncell+1) offsets into pts; self: index of the query in pts.
RGS_HD float rgs_knn3(const RgsKnnGrid& g, const float* pts, const int* cell_start, int64_t n, int64_t self) {
    const float px = pts[3 * self], py = pts[3 * self + 1], pz = pts[3 * self + 2];
    int c[3];
    const float p[3] = {px, py, pz};
    for (int a = 0; a < 3; ++a) {
        int v = (int)floorf((p[a] - g.lo[a]) / g.cell);
        c[a] = v < 0 ? 0 : (v >= g.dims[a] ? g.dims[a] - 1 : v);
    }
    float best[3] = {3.0e38f, 3.0e38f, 3.0e38f};
    const int rmax = rgs_imax(g.dims[0], rgs_imax(g.dims[1], g.dims[2]));
    for (int r = 0; r <= rmax; ++r) {
        for (int dz = -r; dz <= r; ++dz) {
            const int z = c[2] + dz;
            if (z < 0 || z >= g.dims[2]) continue;
            for (int dy = -r; dy <= r; ++dy) {
                const int y = c[1] + dy;
                if (y < 0 || y >= g.dims[1]) continue;
                const bool shell_yz = (dz == -r || dz == r || dy == -r || dy == r);
                for (int dx = -r; dx <= r; dx += (shell_yz || r == 0) ? 1 : 2 * r) {
                    const int x = c[0] + dx;
                    if (x < 0 || x >= g.dims[0]) continue;
                    const int64_t cid = ((int64_t)x * g.dims[1] + y) * g.dims[2] + z;
                    for (int64_t j = cell_start[cid]; j < cell_start[cid + 1]; ++j) {
                        if (j == self) continue;
                        const float ex = pts[3 * j] - px, ey = pts[3 * j + 1] - py, ez = pts[3 * j + 2] - pz;
                        rgs_knn_insert(ex * ex + ey * ey + ez * ez, best);
                    }
                }
            }
        }
        // everything inside the visited block of cells is known; the nearest unvisited point is at least `reach` away
        float reach = 3.0e38f;
        bool covers_all = true;
        for (int a = 0; a < 3; ++a) {
            const float cl = g.lo[a] + (c[a] - r) * g.cell, ch = g.lo[a] + (c[a] + r + 1) * g.cell;
            if (c[a] - r > 0) { reach = fminf(reach, p[a] - cl); covers_all = false; }
            if (c[a] + r < g.dims[a] - 1) { reach = fminf(reach, ch - p[a]); covers_all = false; }
        }
        if (covers_all) break;
        if (reach > 0.0f && best[2] <= reach * reach) break;
    }
    const int64_t others = n - 1;
    if (others <= 0) return 0.0f;
    if (others == 1) return best[0];
    if (others == 2) return 0.5f * (best[0] + best[1]);
    return (best[0] + best[1] + best[2]) / 3.0f;
}
