/* Bullet-chip decals on the walls (engine.py:13747-13991).
 * Part of gd_render.cu (one translation unit); not meant to be included elsewhere.
 *
 * A lane carries a ring of decal slots (engine.py:1870-1884).  The chips in use are
 * projected by threads over slots, the ones that face the viewer and reach the screen are
 * listed and ranked by serial number (the reference paints old to new, 13763-13795), and
 * thread x then shades column x of every listed chip in that order, onto the pixels
 * whose surface depth equals the chip's own ray depth (13950).
 *
 * The reference keeps a depth buffer; this kernel has none.  The surface a pixel shows is
 * recovered from what the walk recorded for its column: rows drawn by a wall tier belong
 * to the first clip event whose textured tier range holds them (tiers only ever draw rows
 * no earlier tier drew, 12687) and have that crossing's distance (12872); of the other rows,
 * those a visplane mark claimed first have the plane's depth (13372-13412); a two-sided
 * middle texture drawn later overrides both with its own distance (13740).  Rows that
 * only the per-pixel flat fallback filled (no seg and no mark claimed them) are floor or
 * ceiling at the fallback's own depth and are left alone.
 */
#ifndef GD_DECALS_CUH
#define GD_DECALS_CUH

struct __align__(16) GdDecalProj {
  float lx, ly, segx, segy;      /* the chip's left end on the map and its extent */
  float zTop;                    /* impact height + top offset * scale */
  int serial;
  short sl, sr;                  /* screen columns [sl, sr) */
  short light;                   /* sector light + fake contrast + weapon flash */
  unsigned short slotStyle;      /* slot (10 bits) | variant << 10 | mirrored << 13 | upside down << 14 */
};
static_assert(sizeof(GdDecalProj) == 32, "scratch layout");

__host__ __device__ inline size_t gd_decal_scratch_per_cta(int slots) {
  return gd_align16((size_t)slots * sizeof(GdDecalProj));
}

__device__ __noinline__ void gd_decals(const GdScene &sc_, const GdView &v_, const GdShared &sh_, const GdEvent *events,
                                       const int *eventCount, const gd_decal *ring, int slots, uint8_t *scratch) {
  const GdScene &sc = *gd_as_shared(&sc_);
  const GdView &v = *gd_as_shared(&v_);
  const GdShared &sh = *gd_as_shared(&sh_);
  const int tid = threadIdx.x;
  int *count = &sh.misc[12];
  GdDecalProj *proj = (GdDecalProj *)scratch;
  if (tid == 0) *count = 0;
  __syncthreads();
  const float width = (float)sc.decalW;
  /* ---- project the chips in use (engine.py:13797-13883) ---- */
  for (int s = tid; s < slots; s += GD_THREADS) {
    const int4 raw = *reinterpret_cast<const int4 *>(&ring[s]);
    const int serial = raw.x;
    if (serial < 0) continue;
    const int w = min(max((int)(short)(raw.y & 0xFFFF), 0), sc.W - 1);
    const int style = (raw.y >> 16) & 0xFFFF;
    const float alongWall = __int_as_float(raw.z), impactZ = __int_as_float(raw.w);
    const int variant = style % 5, flipX = (style / 5) % 2, flipY = (style / 10) % 2, side = style / 20;
    if (variant >= sc.decals || side > 1) continue;
    const float4 wl = *reinterpret_cast<const float4 *>(&sc.walls[w * 4]);
    const float vecx = wl.z - wl.x, vecy = wl.w - wl.y;
    const float cross = vecx * (v.y - wl.y) - vecy * (v.x - wl.x);
    if ((cross > 0 ? 1 : 0) != side) continue;       /* the chip is on the far side of its line */
    const float impx = wl.x + alongWall * vecx, impy = wl.y + alongWall * vecy;
    const int fine = sc.wallFine[w * 2 + side] & 8191;
    const float tanx = (float)sc.fineSine[(fine + 2048) & 8191] / 65536.0f, tany = (float)sc.fineSine[fine] / 65536.0f;
    const int4 info = *reinterpret_cast<const int4 *>(&sc.decalInfo[variant * 4]);   /* height, left, top */
    const float leftOff = (float)info.y, topOff = (float)info.z;
    const float a = leftOff * GD_DECAL_SCALE, b = (width - leftOff) * GD_DECAL_SCALE;
    const float lx = impx - tanx * a, ly = impy - tany * a;
    const float rx = impx + tanx * b, ry = impy + tany * b;
    const i64 ex[2] = {gd_rint(lx * 65536.0f), gd_rint(rx * 65536.0f)};
    const i64 ey[2] = {gd_rint(ly * 65536.0f), gd_rint(ry * 65536.0f)};
    i64 tx[2], ty[2];
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      const i64 relx = ex[e] - v.vx, rely = ey[e] - v.vy;
      tx[e] = (relx * v.vsin - rely * v.vcos) >> 20;
      ty[e] = (relx * v.vcos + rely * v.vsin) >> 20;
    }
    const i64 cf = 160 * GD_FU;
    const i64 sty1 = ty[0] == 0 ? 1 : ty[0], sty2 = ty[1] == 0 ? 1 : ty[1];
    const i64 pl = ((cf + gd_div(tx[0] * cf, sty1)) >> 16) + (tx[0] >= 0);
    const i64 pr = ((cf + gd_div(tx[1] * cf, sty2)) >> 16) + (tx[1] >= 0);
    const i64 lden = tx[0] - tx[1] - ty[1] + ty[0], rden = ty[1] - ty[0] - tx[1] + tx[0];
    const bool leftInside = tx[0] >= -ty[0] && tx[0] <= ty[0] && ty[0] != 0;
    const bool rightInside = tx[1] <= ty[1] && tx[1] >= -ty[1] && ty[1] != 0;
    const bool leftClipped = tx[0] < -ty[0] && tx[1] >= -ty[1] && lden != 0;
    const bool rightClipped = tx[1] > ty[1] && tx[0] <= ty[0] && rden != 0;
    const i64 screenL = leftInside ? gd_clamp(pl, 0, GD_SW) : 0, screenR = rightInside ? gd_clamp(pr, 0, GD_SW) : GD_SW;
    if (!((leftInside || leftClipped) && (rightInside || rightClipped) && screenR > screenL)) continue;
    int sector = gd_wsec(sc, w * 2 + side);
    if (sector < 0) sector = 0;
    const bool horizontal = fabsf(vecy) < 1e-6f, vertical = fabsf(vecx) < 1e-6f;
    GdDecalProj out;
    out.lx = lx; out.ly = ly; out.segx = rx - lx; out.segy = ry - ly;
    out.zTop = impactZ + topOff * GD_DECAL_SCALE;
    out.serial = serial;
    out.sl = (short)screenL; out.sr = (short)screenR;
    out.light = (short)(gd_sec_info(sc, sector).x + (vertical ? 16 : (horizontal ? -16 : 0)) + v.flashLight * 16);
    out.slotStyle = (unsigned short)(s | (variant << 10) | (flipX << 13) | (flipY << 14));
    proj[atomicAdd(count, 1)] = out;
  }
  __syncthreads();
  const int n = *count;
  if (n == 0) return;                                /* block-uniform */
  /* ---- oldest first (engine.py:13763-13775); the ranked list and every chip's column span go to
   * shared memory (the hit cache is idle here), so a column rejects the chips beside it cheaply ---- */
  short *ranked = (short *)sh.hitD;                  /* GD_MAX_DECAL_SLOTS x 2 bytes */
  unsigned *spans = (unsigned *)sh.hitA;             /* GD_MAX_DECAL_SLOTS x 4 bytes: first column | end column << 16 */
  static_assert(GD_MAX_DECAL_SLOTS * 4 <= 8 * GD_SW * 4, "the chip list fits the hit cache");
  for (int i = tid; i < n; i += GD_THREADS) {
    const int si = proj[i].serial, li = proj[i].slotStyle & 1023;
    int rank = 0;
    for (int j = 0; j < n; ++j) {
      const int sj = proj[j].serial;
      rank += (sj < si) || (sj == si && (proj[j].slotStyle & 1023) < li);
    }
    ranked[rank] = (short)i;
    spans[rank] = (unsigned)proj[i].sl | ((unsigned)proj[i].sr << 16);
  }
  __syncthreads();
  /* ---- column x of every listed chip ---- */
  const int x = tid;
  float rx, ry;
  gd_ray(v, x, rx, ry);
  const i64 pitchIndex = gd_clamp((GD_ANG90 - v.pitchBam) >> 19, 0, 4095);
  const float center = 104.0f + (float)(((i64)sc.fineTan[pitchIndex] * 12582912LL) >> 16) / 65536.0f;   /* 13785-13789 */
  const float flatCenter = (103.0f + (float)(((i64)sc.fineTan[pitchIndex] * 12582912LL) >> 16) / 65536.0f) + 0.5f;
  const int nEvents = eventCount[x];
  const bool haveMasked = sc.M > 0 && isfinite(sh.maskedDist[x]);
  const int maskedA = haveMasked ? (int)(sh.maskedInfo[x] & 255u) : 0, maskedB = haveMasked ? (int)((sh.maskedInfo[x] >> 8) & 255u) : 0;
  const float maskedDepth = haveMasked ? sh.maskedDist[x] : GD_INF;
#pragma unroll 1
  for (int k = 0; k < n; ++k) {
    const unsigned span = spans[k];
    if (x < (int)(span & 0xFFFFu) || x >= (int)(span >> 16)) continue;
    const GdDecalProj &d = proj[ranked[k]];
    const int variant = (d.slotStyle >> 10) & 7;
    const bool mirrored = (d.slotStyle >> 13) & 1, upsideDown = (d.slotStyle >> 14) & 1;
    const float den = rx * d.segy - ry * d.segx;
    if (fabsf(den) < 1e-6f) continue;
    const float offx = d.lx - v.x, offy = d.ly - v.y;
    const float distance = (offx * d.segy - offy * d.segx) / den;
    const float along = (offx * ry - offy * rx) / den;
    if (!(distance > 0)) continue;
    int u = (int)gd_clamp((i64)floorf(along * width), 0, sc.decalW - 1);
    if (mirrored) u = sc.decalW - 1 - u;
    const float safeDist = fmaxf(distance, 1e-6f);
    const float vscale = 96.0f / safeDist;
    const float top = center - (d.zTop - v.viewZ) * 192.0f / safeDist;
    const int height = sc.decalInfo[variant * 4];
    /* the rows whose texel row floor((y - top) / vscale) lies in [0, height): a margin of two
     * rows either way, each row then decided by the formula itself */
    const float firstRow = fmaxf(floorf(top) - 2.0f, 0.0f), lastRow = fminf(top + (float)height * vscale + 2.0f, (float)(GD_VH - 1));
    if (!(firstRow <= lastRow)) continue;            /* also a NaN top */
    const i64 depthFixed = gd_rint(safeDist * 4096.0f);
    const int shade = gd_wall_shade(d.light, gd_div(GD_WALL_VIS << 12, gd_max(depthFixed, 1)));
    const uint8_t *opacityRow = sc.decalOpacity + shade * 256;
    const uint8_t *chip = sc.decalAtlas + (size_t)variant * sc.decalH * sc.decalW + u;
    /* rows of this column drawn by a wall tier, and those of them drawn at the chip's depth; only the
     * 32-row words the chip reaches are replayed */
    unsigned tierRows[7] = {0, 0, 0, 0, 0, 0, 0}, chipRows[7] = {0, 0, 0, 0, 0, 0, 0};
    const int word0 = (int)firstRow >> 5, word1 = (int)lastRow >> 5;
#pragma unroll 1
    for (int e = 0; e < nEvents; ++e) {
      const GdEvent ev = events[e * GD_SW + x];
      const bool lower = (ev.pad0 & 2) && ev.t1a < ev.t1b, upper = (ev.pad0 & 1) && ev.t0a < ev.t0b;
      if (!lower && !upper) continue;
      const bool atDepth = fabsf(ev.dist - distance) <= 1e-3f;
#pragma unroll 1
      for (int q = word0; q <= word1; ++q) {
        const unsigned under = gd_range_word(q, ev.t1a, ev.t1b);          /* the lower tier has the row first */
        const unsigned rows = (lower ? under : 0u) | (upper ? gd_range_word(q, ev.t0a, ev.t0b) & ~under : 0u);
        const unsigned fresh = rows & ~tierRows[q];
        tierRows[q] |= fresh;
        if (atDepth) chipRows[q] |= fresh;
      }
    }
    const bool maskedAtDepth = haveMasked && fabsf(maskedDepth - distance) <= 1e-3f;
#pragma unroll 1
    for (int y = (int)firstRow; y <= (int)lastRow; ++y) {
      int tv = (int)gd_clamp((i64)floorf(((float)y - top) / vscale), -1, height);
      if (tv < 0 || tv >= height) continue;
      if (upsideDown) tv = height - 1 - tv;
      const uint8_t src = chip[tv * sc.decalW];
      if (!src) continue;
      bool owns;
      if (haveMasked && y >= maskedA && y < maskedB) {
        owns = maskedAtDepth;
      } else if ((tierRows[y >> 5] >> (y & 31)) & 1u) {
        owns = (chipRows[y >> 5] >> (y & 31)) & 1u;
      } else {
        /* a visplane row: the first event whose floor or ceiling mark holds it (engine.py:12637-12655) */
        owns = false;
#pragma unroll 1
        for (int e = 0; e < nEvents; ++e) {
          const GdEvent ev = events[e * GD_SW + x];
          const bool inFloor = y >= ev.floorA && y < ev.floorB, inCeil = y >= ev.ceilA && y < ev.ceilB;
          if (!(inFloor || inCeil) || ev.sector < 0) continue;
          const float ph = inFloor ? (v.viewZ - gd_sec_floor(sc, ev.sector)) : (gd_sec_ceil(sc, ev.sector) - v.viewZ);
          const float planeDepth = ph * 192.0f / fmaxf(fabsf((float)y - flatCenter), 0.5f);
          owns = fabsf(planeDepth - distance) <= 1e-3f;
          break;
        }
      }
      if (!owns) continue;
      uint8_t *px = sh.frame + y * GD_SW + x;
      *px = sc.decalBlack[min((int)opacityRow[src], 64) * 256 + *px];   /* the table has 65 rows */
    }
  }
  __syncthreads();                                   /* the chip list leaves the hit cache to the sprite pass */
}

#endif
