// Rasterisation: the order in which a persistent grid visits output tiles.
// Plain integer code shared by the kernel and the host (which exposes it for
// tests), so it compiles with or without CUDA.
//
// The five orders carry the numbers the reference's `walk` configuration key
// uses (opengemm/src/mm/types.cuh:78-84, opengemm/src/mm/ptx.cuh:22-119):
//   0  bands `group` tiles wide along N, N fastest inside a band
//   1  the same, every other band walked from the last M row back (serpentine)
//   2  inside a band, blocks of `group` M rows, M fastest inside a block
//   3  a generalised Hilbert curve over the whole tiles_m x tiles_n rectangle
//   4  bands `group` tiles tall along M, M fastest inside a band
// Concurrently running clusters hold consecutive tile numbers, so each order
// decides which operand panels they share in L2.
#pragma once

#if defined(__CUDACC__)
#define OG_HD __host__ __device__ __forceinline__
#else
#define OG_HD inline
#endif

namespace og {

struct TileCoord {
  int mi, ni;
};

enum Walk : int { WALK_BANDS = 0, WALK_SERPENTINE = 1, WALK_BLOCKS = 2, WALK_HILBERT = 3, WALK_ROW_BANDS = 4 };

OG_HD int raster_sign(int v) { return (v > 0) - (v < 0); }
OG_HD int raster_abs(int v) { return v < 0 ? -v : v; }
OG_HD int raster_half(int v) { return v >= 0 ? v / 2 : -((1 - v) / 2); }  // floor(v / 2)

// Position `index` along the generalised Hilbert curve that fills a
// `width` x `height` rectangle (Cerveny's construction for arbitrary sides):
// a rectangle spanned by a major axis A and a minor axis B is cut either in
// two along A (when it is much longer than wide) or into three pieces walked
// B-first, A-second, B-back; the descent follows the piece holding `index`.
OG_HD void hilbert_point(int index, int width, int height, int* px, int* py) {
  int x = 0, y = 0;
  int ax = width >= height ? width : 0, ay = width >= height ? 0 : height;
  int bx = width >= height ? 0 : width, by = width >= height ? height : 0;
  int done = 0;  // curve positions before the current rectangle
  while (true) {
    const int len_a = raster_abs(ax + ay), len_b = raster_abs(bx + by);
    const int sax = raster_sign(ax), say = raster_sign(ay), sbx = raster_sign(bx), sby = raster_sign(by);
    if (len_b == 1) {  // a single row along A
      *px = x + sax * (index - done);
      *py = y + say * (index - done);
      return;
    }
    if (len_a == 1) {
      *px = x + sbx * (index - done);
      *py = y + sby * (index - done);
      return;
    }
    int hax = raster_half(ax), hay = raster_half(ay), hbx = raster_half(bx), hby = raster_half(by);
    if (2 * len_a > 3 * len_b) {
      // long rectangle: two halves along A, the first of even length
      if ((raster_abs(hax + hay) & 1) && len_a > 2) hax += sax, hay += say;
      const int first = raster_abs(hax + hay) * len_b;
      if (index - done < first) {
        ax = hax, ay = hay;
      } else {
        done += first;
        x += hax, y += hay;
        ax -= hax, ay -= hay;
      }
      continue;
    }
    if ((raster_abs(hbx + hby) & 1) && len_b > 2) hbx += sbx, hby += sby;
    const int first = raster_abs(hbx + hby) * raster_abs(hax + hay);
    if (index - done < first) {  // near corner, walked with the axes exchanged
      ax = hbx, ay = hby;
      bx = hax, by = hay;
      continue;
    }
    done += first;
    const int second = len_a * raster_abs((bx - hbx) + (by - hby));
    if (index - done < second) {  // the far strip, full length of A
      x += hbx, y += hby;
      bx -= hbx, by -= hby;
      continue;
    }
    done += second;
    // the remaining corner, walked back towards the start with both axes reversed
    x += (ax - sax) + (hbx - sbx);
    y += (ay - say) + (hby - sby);
    const int rax = -hbx, ray = -hby, rbx = -(ax - hax), rby = -(ay - hay);
    ax = rax, ay = ray, bx = rbx, by = rby;
  }
}

// Tile number -> (M index, N index) for a tiles_m x tiles_n grid.
OG_HD TileCoord tile_coord_of(int tile, int tiles_m, int tiles_n, int group, int walk) {
  if (walk == WALK_HILBERT) {
    TileCoord t;
    hilbert_point(tile, tiles_m, tiles_n, &t.mi, &t.ni);
    return t;
  }
  if (walk == WALK_ROW_BANDS) {
    const int band_tiles = tiles_n * group;
    const int band = tile / band_tiles;
    const int first = band * group;
    const int height = group < tiles_m - first ? group : tiles_m - first;
    const int in_band = tile - band * band_tiles;
    return {first + in_band % height, in_band / height};
  }
  const int band_tiles = tiles_m * group;
  const int band = tile / band_tiles;
  const int first = band * group;
  const int width = group < tiles_n - first ? group : tiles_n - first;
  int in_band = tile - band * band_tiles;
  if (walk == WALK_BLOCKS) {
    const int block = in_band / (group * width);
    const int first_m = block * group;
    const int height = group < tiles_m - first_m ? group : tiles_m - first_m;
    in_band -= block * group * width;
    return {first_m + in_band % height, first + in_band / height};
  }
  int mi = in_band / width;
  if (walk == WALK_SERPENTINE && (band & 1)) mi = tiles_m - 1 - mi;
  return {mi, first + in_band % width};
}

}  // namespace og
