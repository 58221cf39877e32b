/* Area resize to the observation, shared-memory staging of the scene tables, the per-lane palette.
 * Part of gd_render.cu (one translation unit); not meant to be included elsewhere. */
#ifndef GD_OUTPUT_CUH
#define GD_OUTPUT_CUH

/* ---- phase: 320x240 -> 84x84 area resize + grayscale ---------------------
 * Integer definition: src/gradoom/_triton_kernels.py:120-177.  The weights
 * (y_overlap*x_overlap)/48 factor exactly into (y_overlap/12)*(x_overlap/4). */
__device__ void gd_resize(const uint8_t *frame, const unsigned long long *pal64, int srcRows, uint8_t *out) {
  frame = gd_as_shared(frame); pal64 = gd_as_shared(pal64); out = gd_as_shared(out);
  for (int o = threadIdx.x; o < GD_OBS * GD_OBS; o += GD_THREADS) {
    int oy = o / GD_OBS, ox = o - oy * GD_OBS;
    int ys = oy * 240, ye = ys + 240, xs = ox * 320, xe = xs + 320;
    /* An output pixel overlaps at most 4 source rows and 5 source columns; taps
     * past the overlap get weight zero, so the tap loops have fixed trip counts
     * and their loads are independent. */
    const int sy0 = ys / 84, sx0 = xs / 84;
    if (sy0 >= srcRows) { out[o] = 0; continue; }    /* only masked status-bar rows: black */
    unsigned wx[5];
    int cx[5];
#pragma unroll
    for (int j = 0; j < 5; ++j) {
      int sx = sx0 + j;
      int xo = min(xe, (sx + 1) * 84) - max(xs, sx * 84);
      wx[j] = xo > 0 ? (unsigned)xo / 4u : 0u;
      cx[j] = min(sx, GD_SW - 1);
    }
    unsigned long long acc = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      int sy = sy0 + i;
      int yo = min(ye, (sy + 1) * 84) - max(ys, sy * 84);
      unsigned wy = (yo > 0 && sy < srcRows) ? (unsigned)yo / 12u : 0u;
      const uint8_t *row = frame + min(sy, srcRows - 1) * GD_SW;      /* rows beyond srcRows weigh nothing */
      unsigned long long racc = 0;
#pragma unroll
      for (int j = 0; j < 5; ++j) racc += (unsigned long long)wx[j] * pal64[row[cx[j]]];
      acc += racc * wy;
    }
    unsigned r = (unsigned)(acc & 0xFFFFF), g = (unsigned)((acc >> 20) & 0xFFFFF), b = (unsigned)((acc >> 40) & 0xFFFFF);
    r = (r + 800) / 1600; g = (g + 800) / 1600; b = (b + 800) / 1600;
    out[o] = (uint8_t)((r * 77 + g * 150 + b * 29 + 128) >> 8);
  }
}

/* ---- scene tables staged in shared memory ----------------------------------
 * The column walk chases small topology tables (wall endpoints, sector lists,
 * heights) through long dependent chains; from global memory every link costs
 * an L1/L2 round trip.  Each CTA therefore copies the tables that fit into its
 * shared memory once per launch, in this priority order, and redirects the
 * scene's pointers to the copies. */
enum {
  GD_STAGE_WALLS = 1, GD_STAGE_WSEC = 2, GD_STAGE_SECLIST = 4, GD_STAGE_SECTORS = 8, GD_STAGE_WVTX = 16,
  GD_STAGE_WLEN = 32, GD_STAGE_SIDETEX = 64, GD_STAGE_SIDEOFF = 128, GD_STAGE_VTXLIST = 256, GD_STAGE_ROWPROJ = 512
};

__host__ __device__ inline size_t gd_stage_bytes(int bit, int W, int S, int V, int secWallsN, int vtxWallsN) {
  switch (bit) {
    case GD_STAGE_WALLS: return gd_align16((size_t)W * 16);
    case GD_STAGE_WSEC: return gd_align16((size_t)W * 8);
    case GD_STAGE_SECLIST: return gd_align16((size_t)(S + 1) * 4) + gd_align16((size_t)(secWallsN > 0 ? secWallsN : 1) * 4);
    case GD_STAGE_SECTORS: return gd_align16((size_t)S * 8) + gd_align16((size_t)S * 16);
    case GD_STAGE_WVTX: return gd_align16((size_t)W * 8);
    case GD_STAGE_WLEN: return gd_align16((size_t)W * 4);
    case GD_STAGE_SIDETEX: return gd_align16((size_t)W * 24);
    case GD_STAGE_SIDEOFF: return gd_align16((size_t)W * 16);
    case GD_STAGE_VTXLIST: return gd_align16((size_t)(V + 1) * 4) + gd_align16((size_t)(vtxWallsN > 0 ? vtxWallsN : 1) * 4);
    case GD_STAGE_ROWPROJ: return gd_align16((size_t)W * 4 * sizeof(GdRowProj));
  }
  return 0;
}

__device__ inline const void *gd_stage_copy(uint8_t *&cursor, const void *src, size_t bytes) {
  uint8_t *dst = cursor;
  const unsigned *s4 = (const unsigned *)src;
  unsigned *d4 = (unsigned *)dst;
  for (size_t i = threadIdx.x; i < bytes / 4; i += GD_THREADS) d4[i] = s4[i];
  cursor += gd_align16(bytes);
  return dst;
}

/* PLAYPAL of the lane in shared memory, as bytes and as packed 3 x 20-bit
 * words for the resize: the scene's palette, or its bonus / damage blends when
 * the lane's flags ask for screen flashes (engine.py:15381-15398; float32,
 * separately rounded, truncating conversion). */
__device__ void gd_lane_palette(const GdScene &sc, const GdShared &sh, int flags) {
  const int i = threadIdx.x;
  if (i >= 256) return;
  float bonus = 0.0f, flash = 0.0f;
  const bool blend = (flags & 4) != 0;
  if (blend) {
    int damage = min((flags >> 8) & 0xFF, 113), bonusCount = (flags >> 16) & 0xFF;
    bonus = fminf((float)bonusCount * 8.0f, 128.0f) / 255.0f;
    flash = sc.damageAlpha[damage] / 255.0f;
  }
  const float gold[3] = {215.0f, 186.0f, 69.0f}, red[3] = {255.0f, 0.0f, 0.0f};
  unsigned ch[3];
#pragma unroll
  for (int c = 0; c < 3; ++c) {
    unsigned v = sc.playpal[i * 3 + c];
    if (blend) {
      float rgb = (float)v * (1.0f - bonus) + gold[c] * bonus;
      float out = rgb * (1.0f - flash) + red[c] * flash;
      out = fminf(fmaxf(out, 0.0f), 255.0f);
      v = (unsigned)out;
    }
    ch[c] = v;
    sh.playpal[i * 3 + c] = (uint8_t)v;
  }
  sh.pal64[i] = (unsigned long long)ch[0] | ((unsigned long long)ch[1] << 20) | ((unsigned long long)ch[2] << 40);
  sh.pal32[i] = ch[0] | (ch[1] << 8) | (ch[2] << 16);
}

#endif
