// Index arithmetic of the RainFusion window permutation, shared by the kernels that move, pool or
// read tokens in the permuted order.
#pragma once

namespace sdb {

// Geometry of the window permutation of a (t, h, w) latent grid with txt_len text tokens.
// Source order:   [text | image in (t, h, w) raster order]
// Permuted order: [image, windows of 8x8 per frame | text]
// When h or w is not a multiple of 8 the first frame stays in raster order and every later frame
// is laid out as: full 8x8 windows, then the h-remainder rows (full width), then the w-remainder
// columns of the windowed rows.
struct Grid {
    int t, h, w, txt;
    int hw, img;        // tokens per frame, image tokens
    int hm, wm, rh, rw; // windowed extent and remainders
    int aligned;
};

__host__ __device__ inline Grid make_grid(int t, int h, int w, int txt) {
    Grid g;
    g.t = t; g.h = h; g.w = w; g.txt = txt;
    g.hw = h * w;
    g.img = t * h * w;
    g.rh = h % 8; g.rw = w % 8;
    g.hm = h - g.rh; g.wm = w - g.rw;
    g.aligned = (g.rh == 0 && g.rw == 0);
    return g;
}

// Source token (index into the source order) that lands at position p of the permuted order.
__device__ __forceinline__ int source_of(const Grid& g, int p) {
    if (p >= g.img) return p - g.img;  // text: back of the permuted order, front of the source
    const int f = p / g.hw;
    const int r = p - f * g.hw;
    int y, x;
    if (!g.aligned && f == 0) {
        return g.txt + p;
    }
    const int win_area = g.hm * g.wm;
    if (r < win_area) {
        const int wpr = g.wm >> 3;  // windows per row of windows
        const int win = r >> 6, in = r & 63;
        const int wy = win / wpr, wx = win - wy * wpr;
        y = wy * 8 + (in >> 3);
        x = wx * 8 + (in & 7);
    } else if (r < win_area + g.rh * g.w) {
        const int r2 = r - win_area;
        y = g.hm + r2 / g.w;
        x = r2 % g.w;
    } else {
        const int r3 = r - win_area - g.rh * g.w;
        y = r3 / g.rw;
        x = g.wm + r3 % g.rw;
    }
    return g.txt + f * g.hw + y * g.w + x;
}

// True if every run of eight consecutive positions of the permuted order (starting at a multiple of
// eight) is a run of eight consecutive source tokens: then a kernel can fetch the permuted order with
// eight-token copies of the un-permuted tensor.  It holds when the width is a multiple of 8 (no
// column remainder) and the text length is too; the row remainder and the raster-order first frame
// are runs of whole rows.
__host__ __device__ inline bool groups_of_eight_are_contiguous(const Grid& g) {
    return g.rw == 0 && g.txt % 8 == 0;
}

}  // namespace sdb
