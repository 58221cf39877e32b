/* Visplane rows, the per-column portal walk with its wall tiers and plane marks, two-sided middle textures.
 * Part of gd_render.cu (one translation unit); not meant to be included elsewhere. */
#ifndef GD_WALK_CUH
#define GD_WALK_CUH

/* ---- visplane rows (engine.py:10879-10954, 10588-10616, 13372-13405) ---- */
struct GdPlaneSpan {
  i64 basex, basey, pviewx, pviewy, phf, gv, shadeBase;
  const uint8_t *tex;
  int wbits, hbits, texW;
  bool narrow;   /* the row's light term fits 32-bit arithmetic (see gd_plane_pixel) */
};

/* Column-independent part of a span setup, one entry per (sector, floor or
 * ceiling), rebuilt for every lane: the three divisions of R_DrawSpan's setup
 * leave the per-crossing path. */
struct GdPlaneEntry {
  i64 phf, gv, shadeBase, xstep, ystep, bx0, by0, pviewx, pviewy;
  const uint8_t *tex;
  int wbits, hbits;
};

static_assert(sizeof(GdPlaneEntry) == GD_PLANE_ENTRY_BYTES, "scratch layout");

__device__ __noinline__ void gd_plane_entry_setup(const GdScene &sc_, const GdView &v_, int sector, bool isFloor,
                                                  GdPlaneEntry &e) {
  const GdScene &sc = *gd_as_shared(&sc_);
  const GdView &v = *gd_as_shared(&v_);
  float ph = isFloor ? (v.viewZ - gd_sec_floor(sc, sector)) : (gd_sec_ceil(sc, sector) - v.viewZ);
  int4 si = gd_sec_info(sc, sector);
  int tex = GD_CHECK_INDEX(isFloor ? si.y : si.z, sc.T);
  const int4 ti = *reinterpret_cast<const int4 *>(&sc.texInfo[tex * 4]);
  e.wbits = ti.z; e.hbits = ti.w;
  e.tex = sc.texAtlas + (size_t)tex * sc.texH * sc.texW;
  i64 xscale = 1LL << (32 - e.wbits), yscale = 1LL << (32 - e.hbits);
  i64 fs = v.vsin, fc = v.vcos;
  e.xstep = gd_div(xscale * fs, GD_FOCAL_X);
  e.ystep = gd_div(yscale * fc, GD_FOCAL_X);
  e.bx0 = (xscale * fc) >> 16;
  e.by0 = (yscale * -fs) >> 16;
  e.pviewx = gd_wmul(xscale, v.vx) >> 16;
  e.pviewy = gd_wmul(yscale, -v.vy) >> 16;
  e.phf = gd_rint(ph * 65536.0f);
  e.gv = gd_min(gd_div(GD_FLOOR_VIS << 16, gd_max(e.phf, 1)), (1LL << 31) - 1);
  i64 light = si.x + v.flashLight * 16;
  e.shadeBase = 64 * GD_FU - (light + 12) * (GD_FU / 4);
  /* gv lies in [0, 2^31) by construction; with the screen centre within +-2^30 (any pitch short of
   * +-89.5 degrees) and a shade base that fits an int, the light term of a pixel needs one 32 x 32 -> 64
   * multiply; the flag travels in the spare bits of hbits */
  const bool narrow = v.center > -(1LL << 30) && v.center < (1LL << 30) && e.shadeBase > -(1LL << 31) && e.shadeBase < (1LL << 31);
  e.hbits |= narrow ? 256 : 0;
}

__device__ __forceinline__ void gd_plane_setup(const GdScene &sc, const GdPlaneEntry *table, int sector, bool isFloor,
                                               int x, GdPlaneSpan &p) {
  const GdPlaneEntry &e = table[gd_secidx(sc, sector) * 2 + (isFloor ? 1 : 0)];
  i64 col = (i64)x - 159;
  p.wbits = e.wbits; p.hbits = e.hbits & 255; p.narrow = (e.hbits & 256) != 0; p.texW = sc.texW;
  p.tex = e.tex;
  p.basex = e.bx0 + col * e.xstep;
  p.basey = e.by0 + col * e.ystep;
  p.pviewx = e.pviewx;
  p.pviewy = e.pviewy;
  p.phf = e.phf;
  p.gv = e.gv;
  p.shadeBase = e.shadeBase;
}

/* One visplane pixel (R_DrawSpan, engine.py:10879-10954).  kNarrow: the span's `narrow` flag holds, so
 * |center - y * 65536| < 2^31 and the light term is exact in 32-bit arithmetic: vis = min(gv * rowDist >> 16,
 * 24 * 65536) is 24 * 65536 exactly when the 64-bit product is at least 0x18 << 32. */
template <bool kNarrow>
__device__ __forceinline__ unsigned gd_plane_pixel(const GdPlaneSpan &p, i64 center, unsigned yslope, unsigned colormap, int y) {
  i64 distance = gd_wmul(p.phf, (i64)gd_lds32(yslope + y * 4)) >> 16;
  i64 xfrac = ((gd_wmul(distance, p.basex) >> 16) + p.pviewx) & GD_U32MASK;
  i64 yfrac = ((gd_wmul(distance, p.basey) >> 16) + p.pviewy) & GD_U32MASK;
  int u = (int)(xfrac >> (32 - p.wbits)), tv = (int)(yfrac >> (32 - p.hbits));
  uint8_t texel = p.tex[tv * p.texW + u];
  int shade;
  if (kNarrow) {
    const int rowDist = abs((int)center - (y << 16));
    const i64 vis64 = (i64)(int)p.gv * (i64)rowDist;
    const int vis = (unsigned)(vis64 >> 32) >= 0x18u ? 24 * 65536 : (int)(unsigned)(vis64 >> 16);
    shade = min(max(((int)p.shadeBase - vis) >> 16, 0), 31);
  } else {
    i64 rowDist = center - (i64)y * GD_FU;
    if (rowDist < 0) rowDist = -rowDist;
    i64 vis = gd_min(gd_wmul(p.gv, rowDist) >> 16, 24 * GD_FU);
    shade = (int)gd_clamp((p.shadeBase - vis) >> 16, 0, 31);
  }
  return gd_lds8(colormap + shade * 256 + texel);
}

/* The 208-row column masks live in shared memory, one word column per screen
 * column: word k of column x is m[k * GD_SW]. */
/* bits of mask word k (rows 32k..32k+31) that lie in rows [a,b) */
__device__ __forceinline__ unsigned gd_range_word(int k, int a, int b) {
  int lo = max(a - (k << 5), 0), hi = min(b - (k << 5), 32);
  if (lo >= hi) return 0u;
  unsigned upto = hi == 32 ? 0xffffffffu : ((1u << hi) - 1u);
  return upto & ~((1u << lo) - 1u);
}

/* rows of line w at column x: fragment aware in the instantiation for scenes with split lines */
template <bool kSplit>
__device__ __forceinline__ int gd_rows(const GdScene &sc, const GdView &v, const GdShared &sh, int w, float worldZ, int x) {
  if (kSplit) return gd_line_rows(sc, v, sh.walls, sh.frags, w, worldZ, x);
  return gd_project_rows(v, sh.walls[w], worldZ, x);
}

/* ---- phase: per-column portal walk (engine.py:11561-13371) -------------- */
struct GdColState {
  int cur;
  int ceilClip, floorClip;
  float prev;
  bool pendOwnerBoundary, pendEpBoundary, pendEpBridgeBoundary, pendPortalBridge;
  float pendOwnerEpX, pendOwnerEpY, pendEpEpX, pendEpEpY;
  int pendEpWall, pendEpBridgeIndex, pendPortalBridgeIndex, pendPortalBridgeSector;
  float pendPortalBridgeExit;
};

__device__ __forceinline__ bool gd_state_equal(const GdColState &a, const GdColState &b) {
  return a.cur == b.cur && a.ceilClip == b.ceilClip && a.floorClip == b.floorClip && a.prev == b.prev &&
         a.pendOwnerBoundary == b.pendOwnerBoundary && a.pendEpBoundary == b.pendEpBoundary &&
         a.pendEpBridgeBoundary == b.pendEpBridgeBoundary && a.pendPortalBridge == b.pendPortalBridge &&
         a.pendOwnerEpX == b.pendOwnerEpX && a.pendOwnerEpY == b.pendOwnerEpY && a.pendEpEpX == b.pendEpEpX &&
         a.pendEpEpY == b.pendEpEpY && a.pendEpWall == b.pendEpWall && a.pendEpBridgeIndex == b.pendEpBridgeIndex &&
         a.pendPortalBridgeIndex == b.pendPortalBridgeIndex &&
         a.pendPortalBridgeSector == b.pendPortalBridgeSector && a.pendPortalBridgeExit == b.pendPortalBridgeExit;
}

/* What one iteration decided for a column; the part other columns of its
 * aligned group of four need is exchanged with shuffles. */
struct GdIter {
  int wall, side;
  bool rasterValid, valid, oneSided;
  int renderCurrent, otherSector;
  float distance;
  i64 vis;
  int ctop, cbot, cupbot, clowtop;
  bool tier[3];
  bool markCeil, markFloor;
  float viewFloor, viewCeil, otherFloor, otherCeil;
  int tex[3];
  /* traversal */
  bool nokpp, pskpp, usesGeo, entersOther, entersShared, endpointOnly, epb, cppb, geometric;
  int nopOther, psOther, gpOther;
  float nopDist, psDist, gpDist, osd;
  bool startsOwner, continuesOwner, pendEpHasFwd;
  float selEpX, selEpY, epEpX, epEpY;
  int epFwdIdx, ppbIdx, psPathIndex;
  bool psFromFront;
};

/* kSplit: the scene has lines a node builder split; the other instantiation carries none of that code */
template <bool kSplit>
__device__ void gd_column_decide(const GdScene &sc_, const GdView &v_, const GdWall *walls, const GdWall *frags,
                                 const unsigned *ownerMask, const GdRowProj *rowproj, float *hitD, float *hitA, uint8_t *hitF, int x, float rx,
                                 float ry, const GdColState &c, GdIter &it) {
  const GdScene &sc = *gd_as_shared(&sc_);
  const GdView &v = *gd_as_shared(&v_);
  walls = gd_as_shared(walls); ownerMask = gd_as_shared(ownerMask);
  hitD = gd_as_shared(hitD); hitA = gd_as_shared(hitA); hitF = gd_as_shared(hitF);
  const int curSector = c.cur;
  const int current = GD_CHECK_SECTOR(curSector < 0 ? 0 : curSector, sc.S);
  const float prev = c.prev;
  const int i0 = sc.secOff[current], i1 = sc.secOff[current + 1];
  /* every rule below looks at the walls of the current sector: test each once
   * and keep the results in this column's slice of shared memory */
  constexpr int kCache = 8;
  const int nCache = min(i1 - i0, kCache);
#pragma unroll 1
  for (int k = 0; k < nCache; ++k) {
    GdHit h = gd_hit(sc, v, walls, GD_CHECK_INDEX(sc.secWalls[i0 + k], sc.W), x, rx, ry);
    hitD[k * GD_SW + x] = h.d;
    hitA[k * GD_SW + x] = h.along;
    hitF[k * GD_SW + x] = (uint8_t)((h.geo ? 1 : 0) | (h.proj ? 2 : 0) | (h.left ? 4 : 0));
  }
  auto loadHit = [&](int k) -> GdHit {
    GdHit h;
    h.d = hitD[k * GD_SW + x];
    h.along = hitA[k * GD_SW + x];
    uint8_t f = hitF[k * GD_SW + x];
    h.geo = f & 1; h.proj = (f & 2) != 0; h.left = (f & 4) != 0;
    return h;
  };
  /* one out-of-line copy of the uncached test serves every rule below */
  auto cachedHit = [&](int w) -> GdHit {
#pragma unroll 1
    for (int k = 0; k < nCache; ++k)
      if (sc.secWalls[i0 + k] == w) return loadHit(k);
    return gd_hit_slow(sc, v, walls, w, x, rx, ry);
  };
#define HIT(w) cachedHit(w)
#define HITK(k) (((k) - i0) < nCache ? loadHit((k) - i0) : gd_hit_slow(sc, v, walls, GD_CHECK_INDEX(sc.secWalls[k], sc.W), x, rx, ry))
  float distance = GD_INF;
  int wallIndex = 0;
  if (curSector >= 0) {
#pragma unroll 1
    for (int k = i0; k < i1; ++k) {
      int w = GD_CHECK_INDEX(sc.secWalls[k], sc.W);
      GdHit h = HITK(k);
      if (h.d > prev && h.d < distance) { distance = h.d; wallIndex = w; }
    }
    float sd = GD_INF;
    int sw = 0;
#pragma unroll 1
    for (int k = i0; k < i1; ++k) {
      int w = GD_CHECK_INDEX(sc.secWalls[k], sc.W);
      if (!walls[w].oneSided) continue;
      GdHit h = HITK(k);
      if (!(h.d > prev) || !isfinite(h.d)) continue;
      if (fabsf(h.d - distance) <= 1e-3f && h.d < sd) { sd = h.d; sw = w; }
    }
    if (isfinite(sd)) { distance = sd; wallIndex = sw; }
  }
  GdHit hSel = HIT(wallIndex);
  const float *selWall = &sc.walls[wallIndex * 4];
  bool selUsesStart = hSel.along <= 0.5f;
  float selEpX = selUsesStart ? selWall[0] : selWall[2], selEpY = selUsesStart ? selWall[1] : selWall[3];
  int selVtx = sc.wvtx[wallIndex * 2 + (selUsesStart ? 0 : 1)];
#define SHARES_SEL(w) (sc.wvtx[(w) * 2] == selVtx || sc.wvtx[(w) * 2 + 1] == selVtx)
  bool continuesOwner = c.pendOwnerBoundary && selEpX == c.pendOwnerEpX && selEpY == c.pendOwnerEpY;
  bool continuesEp = c.pendEpBoundary && selEpX == c.pendEpEpX && selEpY == c.pendEpEpY;
  int selSlot = hSel.along > 0.5f;
  int epFwdIdx = 0;
  bool pendEpHasFwd = false;
  if (continuesEp) {
    bool m = gd_portal_bridge(sc, selSlot, wallIndex, c.pendEpWall, epFwdIdx);
    pendEpHasFwd = m && (HIT(epFwdIdx).d > distance + 1e-3f);
  }
  bool completesPendEpBridge = c.pendEpBridgeBoundary && wallIndex == c.pendEpBridgeIndex;
  bool selIsProjected = hSel.proj;
  bool selExclRight = walls[wallIndex].sr == x;
  float psPathDist = distance;
  int psPathIndex = wallIndex;
  float psd = GD_INF;
  int psi = 0;
  if (!selIsProjected) {
#pragma unroll 1
    for (int k = i0; k < i1; ++k) {
      int w = GD_CHECK_INDEX(sc.secWalls[k], sc.W);
      if (!walls[w].oneSided || !SHARES_SEL(w)) continue;
      GdHit h = HITK(k);
      if (h.proj && h.left && (h.d > prev + 1e-3f) && h.d < psd) { psd = h.d; psi = w; }
    }
    if (selExclRight) {
      const int32_t *off = selUsesStart ? sc.sbStartOff : sc.sbEndOff;
      const int32_t *idx = selUsesStart ? sc.sbStartIdx : sc.sbEndIdx;
      float sbd = GD_INF;
      int sbi = wallIndex;
#pragma unroll 1
      for (int k = off[wallIndex]; k < off[wallIndex + 1]; ++k) {
        int b = GD_CHECK_INDEX(idx[k], sc.W);
        bool inc = gd_wsec(sc, b * 2) == current || gd_wsec(sc, b * 2 + 1) == current;
        if (!inc || !walls[b].oneSided) continue;
        GdHit h = HIT(b);
        if (h.proj && h.left && (h.d > prev + 1e-3f) && h.d < sbd) { sbd = h.d; sbi = b; }
      }
      if (sbd < psd) { psd = sbd; psi = sbi; }
    }
  }
  bool hasProjectedSolidOwner = isfinite(psd);
  if (hasProjectedSolidOwner) { distance = psd; wallIndex = psi; }
  GdHit hW = (wallIndex == psPathIndex) ? hSel : HIT(wallIndex);
  int seo = wallIndex;
  float sed = hW.d;
  if (!hW.proj) gd_endpoint_owner(sc, v, walls, wallIndex, x, rx, ry, hW, seo, sed);
  bool eoPathIsGeo = hW.geo;
  bool replaceEo = (seo != wallIndex) && (sed > prev + 1e-3f);
  if (replaceEo) { distance = sed; wallIndex = seo; hW = HIT(wallIndex); }
  int nopIndex = wallIndex;
  float nopDist = distance;
  bool nopIsGeo = replaceEo ? eoPathIsGeo : hW.geo;
  bool nopFromFront = curSector == gd_wsec(sc, nopIndex * 2);
  int nopOther = nopFromFront ? gd_wsec(sc, nopIndex * 2 + 1) : gd_wsec(sc, nopIndex * 2);
  bool selOwnerIsProjected = hW.proj;
  bool selOwnerExclRight = walls[wallIndex].sr == x;
  i64 selOwnerSpan = walls[wallIndex].sr - walls[wallIndex].sl;
  bool selOwnerShort = sc.wlen[wallIndex] <= 32.0f;
  float npd = GD_INF;
  int npi = 0;
  if (!selOwnerIsProjected) {
#pragma unroll 1
    for (int k = i0; k < i1; ++k) {
      int w = GD_CHECK_INDEX(sc.secWalls[k], sc.W);
      if (walls[w].oneSided) continue;
      GdHit h = HITK(k);
      if (!h.proj || !(h.d > prev + 1e-3f)) continue;
      bool topological = false;
      if (h.left && selOwnerExclRight && selOwnerSpan <= 2) {
        int sbIdx;
        topological = gd_sector_bridge(sc, h.along > 0.5f, w, nopIndex, sbIdx);
      }
      bool a = gd_same_pair(sc, wallIndex, w) ||
               (h.left && selOwnerExclRight && (selOwnerSpan <= 2 || (SHARES_SEL(w) && selOwnerShort)));
      bool nearOwner = (a && (fabsf(h.d - distance) <= gd_tol(h.d))) || topological;
      if (nearOwner && h.d < npd) { npd = h.d; npi = w; }
    }
  }
  /* projected sector bridge (engine.py:12073-12164) */
  const int pew = c.pendEpWall;
  bool peFromCur = curSector == gd_wsec(sc, pew * 2);
  int peOther = peFromCur ? gd_wsec(sc, pew * 2 + 1) : gd_wsec(sc, pew * 2);
  bool usePsb = false;
  if (c.pendEpBoundary && !selOwnerIsProjected && selOwnerExclRight && nopIsGeo) {
    bool peIncident = peFromCur || curSector == gd_wsec(sc, pew * 2 + 1);
    const float *peWall = &sc.walls[pew * 4];
    int peSlot = (c.pendEpEpX == peWall[2] && c.pendEpEpY == peWall[3]) ? 1 : 0;
    int psbIndex;
    bool psbExists = gd_sector_bridge(sc, peSlot, pew, nopIndex, psbIndex);
    if (psbExists && peIncident && peOther >= 0 && nopOther >= 0 && (walls[pew].sr - walls[pew].sl <= 1)) {
      int b0 = gd_wsec(sc, psbIndex * 2), b1 = gd_wsec(sc, psbIndex * 2 + 1);
      bool matches = (b0 == peOther && b1 == nopOther) || (b1 == peOther && b0 == nopOther);
      GdHit hb = HIT(psbIndex);
      GdHit hp = HIT(pew);
      bool psb = matches && hb.proj && hb.left && (hb.d > prev - gd_tol(hp.d)) && (hb.d < nopDist);
      if (psb && hb.d < npd) { usePsb = true; npd = hb.d; npi = psbIndex; }
    }
  }
  bool replaceNp = isfinite(npd);
  if (replaceNp) { distance = npd; wallIndex = npi; hW = HIT(wallIndex); }
  bool finalIsProjected = hW.proj, finalIsGeo = hW.geo;
  bool completesOpposing =
      c.pendEpBoundary && finalIsProjected && !finalIsGeo && gd_opposing_pair(sc, pew, wallIndex);
  bool valid = isfinite(distance);
  bool boundaryHasOwner = (ownerMask[x >> 5] >> (x & 31)) & 1u;
  bool exclTraversalOnly =
      !selOwnerIsProjected && selOwnerExclRight && !replaceNp && selOwnerSpan <= 2 && !boundaryHasOwner;
  bool rasterValid = valid && !exclTraversalOnly && !continuesOwner &&
                     !((pendEpHasFwd || completesPendEpBridge) && !selIsProjected && selExclRight && !replaceNp);
  bool geometric = replaceNp ? nopIsGeo : (replaceEo ? eoPathIsGeo : hW.geo);
  bool nokpp = replaceNp && nopIsGeo && nopOther >= 0;
  int front = gd_wsec(sc, wallIndex * 2), back = gd_wsec(sc, wallIndex * 2 + 1);
  bool fromFront = curSector == front;
  int otherSector = fromFront ? back : front;
  int renderCurrent = usePsb ? peOther : (completesOpposing ? otherSector : current);
  bool renderFromFront = renderCurrent == front;
  int renderOther = renderFromFront ? back : front;
  int side = renderFromFront ? 0 : 1;
  const GdWall &wv = walls[wallIndex];
  const bool splitLine = kSplit && gd_line_is_split(sc, wallIndex);      /* a node builder cut this line: the slow way */
  i64 vis = splitLine ? gd_line_vis(sc, walls, frags, wallIndex, side, x)
                      : wv.visL[side] + ((i64)x - wv.visSl[side]) * wv.visStep[side];
  bool psFromFront = curSector == gd_wsec(sc, psPathIndex * 2);
  int psOther = psFromFront ? gd_wsec(sc, psPathIndex * 2 + 1) : gd_wsec(sc, psPathIndex * 2);
  bool pskpp = hasProjectedSolidOwner && hSel.geo && psOther >= 0;
  int safeOther = renderOther < 0 ? 0 : renderOther;
  float viewFloor = gd_sec_floor(sc, renderCurrent), viewCeil = gd_sec_ceil(sc, renderCurrent);
  float otherFloor = gd_sec_floor(sc, safeOther), otherCeil = gd_sec_ceil(sc, safeOther);
  bool oneSided = otherSector < 0;
  const int32_t *stex = &sc.sideTex[(wallIndex * 2 + side) * 3];
  /* Row bounds: per (wall, sector height) tables built once per lane cover the
   * usual case of heights taken from the wall's own two sectors. */
  const GdRowProj *rp = rowproj + wallIndex * 4;
  int slotCur = (renderCurrent == front) ? 0 : ((renderCurrent == back && back >= 0) ? 2 : -1);
  int oneTop = 0, oneBottom = 0;
  /* the row bounds feed tiers, marks, clips and events, all of which need a
   * raster-valid crossing */
  if (!rasterValid) {
  } else if (splitLine) {
    oneTop = gd_line_rows(sc, v, walls, frags, wallIndex, viewCeil, x);
    oneBottom = gd_line_rows(sc, v, walls, frags, wallIndex, viewFloor, x);
  } else if (slotCur >= 0) {
    oneBottom = gd_rowproj_eval(v, wv, rp[slotCur], x);
    oneTop = gd_rowproj_eval(v, wv, rp[slotCur + 1], x);
  } else {
    oneTop = gd_project_rows(v, wv, viewCeil, x);
    oneBottom = gd_project_rows(v, wv, viewFloor, x);
  }
  int lowerTop = 0, upperBottom = 0;
  if (!oneSided && rasterValid) {  /* the tiers and clips below use them only for two-sided lines */
    int slotOther = (renderOther >= 0 && renderOther == back) ? 2 : ((renderOther >= 0 && renderOther == front) ? 0 : -1);
    if (splitLine) {
      lowerTop = gd_line_rows(sc, v, walls, frags, wallIndex, otherFloor, x);
      upperBottom = gd_line_rows(sc, v, walls, frags, wallIndex, otherCeil, x);
    } else if (slotOther >= 0) {
      lowerTop = gd_rowproj_eval(v, wv, rp[slotOther], x);
      upperBottom = gd_rowproj_eval(v, wv, rp[slotOther + 1], x);
    } else {
      lowerTop = gd_project_rows(v, wv, otherFloor, x);
      upperBottom = gd_project_rows(v, wv, otherCeil, x);
    }
  }
  int ctop = max(oneTop, c.ceilClip), cbot = min(oneBottom, c.floorClip);
  int cupbot = max(min(upperBottom, c.floorClip), ctop);
  int clowtop = min(max(lowerTop, c.ceilClip), cbot);
  int4 ri = gd_sec_info(sc, renderCurrent), oi = gd_sec_info(sc, safeOther);
  bool lightDiff = ri.x != oi.x;
  it.markCeil = oneSided || viewCeil != otherCeil || ri.z != oi.z || lightDiff;
  it.markFloor = oneSided || viewFloor != otherFloor || ri.y != oi.y || lightDiff;
  it.wall = wallIndex; it.side = side; it.rasterValid = rasterValid; it.valid = valid;
  it.oneSided = oneSided; it.renderCurrent = renderCurrent; it.otherSector = otherSector;
  it.distance = distance; it.vis = vis;
  it.ctop = ctop; it.cbot = cbot; it.cupbot = cupbot; it.clowtop = clowtop;
  it.viewFloor = viewFloor; it.viewCeil = viewCeil; it.otherFloor = otherFloor; it.otherCeil = otherCeil;
  it.tex[0] = stex[0]; it.tex[1] = stex[1]; it.tex[2] = stex[2];
  it.tier[0] = oneSided && rasterValid && stex[0] >= 0 && ctop < cbot;
  it.tier[1] = !oneSided && rasterValid && (viewFloor < otherFloor) && stex[1] >= 0 && clowtop < cbot;
  it.tier[2] = !oneSided && rasterValid && (viewCeil > otherCeil) && stex[2] >= 0 && ctop < cupbot;

  /* traversal decisions (engine.py:13070-13241) */
  bool endpointOnly = valid && !oneSided && !geometric;
  float cnd = GD_INF, ond = GD_INF, csd = GD_INF, osd = GD_INF, gpd = GD_INF;
  int cni = 0, oni = 0, gpi = 0;
  const float prior = prev;
  if (endpointOnly) {
#pragma unroll 1
    for (int k = i0; k < i1; ++k) {
      int w = GD_CHECK_INDEX(sc.secWalls[k], sc.W);
      GdHit h = HITK(k);
      bool os = walls[w].oneSided;
      bool fut = (h.geo || (os && isfinite(h.d))) && (h.d > distance + 1e-3f);
      if (fut && h.d < cnd) { cnd = h.d; cni = w; }
      bool sharesEp = gd_shares_endpoint(sc, w, wallIndex);
      bool sharedSolid = isfinite(h.d) && os && (sharesEp || h.left) && (h.d > prior + 1e-3f) &&
                         (h.d <= distance + 1e-3f);
      if (sharedSolid && h.d < csd) csd = h.d;
      bool sgp = h.geo && sharesEp && !os && (h.d > prior + 1e-3f) && (fabsf(h.d - distance) <= (1.0f / 16.0f));
      if (sgp && h.d < gpd) { gpd = h.d; gpi = w; }
    }
    /* endpointOnly implies otherSector >= 0 */
#pragma unroll 1
    for (int k = sc.secOff[otherSector]; k < sc.secOff[otherSector + 1]; ++k) {
      int w = GD_CHECK_INDEX(sc.secWalls[k], sc.W);
      GdHit h = HIT(w);
      bool os = walls[w].oneSided;
      bool fut = (h.geo || (os && isfinite(h.d))) && (h.d > distance + 1e-3f);
      if (fut && h.d < ond) { ond = h.d; oni = w; }
      bool sharesEp = gd_shares_endpoint(sc, w, wallIndex);
      bool sharedSolid = isfinite(h.d) && os && (sharesEp || h.left) && (h.d > prior + 1e-3f) &&
                         (h.d <= distance + 1e-3f);
      if (sharedSolid && h.d < osd) osd = h.d;
    }
  }
  bool tied = endpointOnly && isfinite(cnd) && cni == oni && gd_opposing_pair(sc, wallIndex, cni);
  bool entersOther = endpointOnly && otherSector >= 0 && ((ond < cnd) || tied);
  bool entersShared = endpointOnly && otherSector >= 0 && (osd < csd);
  bool gpFromFront = curSector == gd_wsec(sc, gpi * 2);
  int gpOther = gpFromFront ? gd_wsec(sc, gpi * 2 + 1) : gd_wsec(sc, gpi * 2);
  bool usesGeo = endpointOnly && isfinite(gpd) && gpOther >= 0;
  int ppbIdx = 0;
  bool epb = false;
  if (usesGeo) {
    GdHit hg = HIT(gpi);
    bool ppbExists = gd_portal_bridge(sc, hg.along > 0.5f, gpi, wallIndex, ppbIdx);
    if (ppbExists) {
      GdHit hb = HIT(ppbIdx);
      epb = hb.proj && hb.left && (hb.d > prior + 1e-3f) && (fabsf(hb.d - gpd) <= gd_tol(hg.d));
    }
  }
  it.cppb = valid && c.pendPortalBridge && wallIndex == c.pendPortalBridgeIndex;
  it.nokpp = nokpp; it.pskpp = pskpp; it.usesGeo = usesGeo; it.entersOther = entersOther;
  it.entersShared = entersShared; it.endpointOnly = endpointOnly; it.epb = epb; it.geometric = geometric;
  it.nopOther = nopOther; it.psOther = psOther; it.gpOther = gpOther;
  it.nopDist = nopDist; it.psDist = psPathDist; it.gpDist = gpd; it.osd = osd;
  it.startsOwner = replaceNp; it.continuesOwner = continuesOwner; it.pendEpHasFwd = pendEpHasFwd;
  it.selEpX = selEpX; it.selEpY = selEpY;
  {
    const float *fw = &sc.walls[wallIndex * 4];
    bool us = hW.along <= 0.5f;
    it.epEpX = us ? fw[0] : fw[2];
    it.epEpY = us ? fw[1] : fw[3];
  }
  it.epFwdIdx = epFwdIdx; it.ppbIdx = ppbIdx; it.psPathIndex = psPathIndex; it.psFromFront = psFromFront;
#undef HIT
#undef HITK
#undef SHARES_SEL
}

/* Draw rows [ya,yb) of one wall tier in column x, skipping rows [ea,eb)
 * (the overlapping lower tier, which has priority) and rows already filled.
 * engine.py:12762-12884. */
struct GdTierCtx {
  i64 hoff, tox, vstepBase, light;
  float yoff;
  int tailBottom;   /* rows >= tailBottom use the group's first-column light; 255+ = never */
};

__device__ __noinline__ void gd_draw_tier(const GdScene &sc_, const GdView &v_, const GdShared &sh_, int x, int ya, int yb, int ea,
                             int eb, int texId, float originZ, const GdTierCtx &t, i64 vis, i64 firstVis,
                             bool tailValid, int tailBottom, int oa, int ob, bool oTailValid, int oTailBottom,
                             unsigned *filled) {
  const GdScene &sc = *gd_as_shared(&sc_);
  const GdView &v = *gd_as_shared(&v_);
  const GdShared &sh = *gd_as_shared(&sh_);
  if (texId < 0 || ya >= yb) return;
#ifdef GD_CHECKED
  if (texId >= sc.T) { atomicOr(gdCheckedStatus, GD_STATUS_BAD_INDEX); return; }   /* the tier stays undrawn */
#endif
  filled = gd_as_shared(filled);
  const int4 ti = *reinterpret_cast<const int4 *>(&sc.texInfo[texId * 4]);
  int tw = ti.x, hbits = ti.w;
  int u = gd_pymod_width((t.hoff + t.tox) >> 16, tw);
  i64 vstep = t.vstepBase * (1LL << (14 - hbits));
  i64 texMid = gd_rint((originZ - v.viewZ) * 65536.0f + t.yoff * 65536.0f);
  /* frac(y) = (texMid << (16-bits)) + ((vstep * (y*FU - center + FU)) >> 16); the
   * y term is a multiple of 2^16 inside the shift, so it steps by vstep exactly. */
  unsigned base = (unsigned)(gd_shl(texMid, 16 - hbits) + (gd_wmul(vstep, GD_FU - v.center) >> 16));
  unsigned step = (unsigned)vstep;
  const uint8_t *col = sc.texAtlasCol + ((size_t)texId * sc.texW + u) * sc.texH;
  int shadeN = gd_wall_shade(t.light, vis), shadeT = gd_wall_shade(t.light, firstVis);
  const unsigned cmN = gd_shared_addr(sh.colormap + shadeN * 256), cmT = gd_shared_addr(sh.colormap + shadeT * 256);
  /* rows lit with the group's first-column light */
  const int tailA = tailValid ? tailBottom : GD_VH, oTailA = oTailValid ? max(oa, oTailBottom) : 0,
            oTailB = oTailValid ? ob : 0;
  const int shift = 32 - hbits;
  const unsigned dst = gd_shared_addr(sh.frame + x);
#pragma unroll 1
  for (int k = ya >> 5; k <= (yb - 1) >> 5; ++k) {
    unsigned have = filled[k * GD_SW];
    unsigned m = gd_range_word(k, ya, yb) & ~gd_range_word(k, ea, eb) & ~have;
    if (!m) continue;
    filled[k * GD_SW] = have | m;
    const unsigned tailM = gd_range_word(k, tailA, GD_VH) | gd_range_word(k, oTailA, oTailB);
    const int y0 = k << 5;
    /* two rows per trip; an odd last row is simply drawn twice */
#pragma unroll 1
    while (m) {
      int b0 = __ffs(m) - 1;
      m &= m - 1;
      int b1 = m ? __ffs(m) - 1 : b0;
      m &= m - 1;
      unsigned f0 = base + (unsigned)(y0 + b0) * step, f1 = base + (unsigned)(y0 + b1) * step;
      const unsigned t0 = col[f0 >> shift], t1 = col[f1 >> shift];
      const unsigned p0 = gd_lds8(((tailM >> b0) & 1u ? cmT : cmN) + t0), p1 = gd_lds8(((tailM >> b1) & 1u ? cmT : cmN) + t1);
      gd_sts8(dst + (y0 + b0) * GD_SW, p0);
      gd_sts8(dst + (y0 + b1) * GD_SW, p1);
    }
  }
}

/* Rows [ya,yb) of column x that no plane owns yet become the span's; those no wall tier filled are drawn.
 * The pointers and the centre are taken into registers first: the byte stores into the frame would make the
 * compiler read them again from the shared structures on every trip. */
template <bool kNarrow>
__device__ __forceinline__ void gd_plane_rows(const GdPlaneSpan &p, i64 center, const GdShared &sh, int x, int ya, int yb,
                                              unsigned *owned, const unsigned *filled) {
  const unsigned dst = gd_shared_addr(sh.frame + x);
  const unsigned yslope = gd_shared_addr(sh.yslope), colormap = gd_shared_addr(sh.colormap);
  owned = gd_as_shared(owned); filled = gd_as_shared(filled);
#pragma unroll 1
  for (int k = ya >> 5; k <= (yb - 1) >> 5; ++k) {
    unsigned have = owned[k * GD_SW];
    unsigned fresh = gd_range_word(k, ya, yb) & ~have;
    if (!fresh) continue;
    owned[k * GD_SW] = have | fresh;
    unsigned m = fresh & ~filled[k * GD_SW];
    const int y0 = k << 5;
#pragma unroll 1
    while (m) {
      int b0 = __ffs(m) - 1;
      m &= m - 1;
      int b1 = m ? __ffs(m) - 1 : b0;
      m &= m - 1;
      const unsigned p0 = gd_plane_pixel<kNarrow>(p, center, yslope, colormap, y0 + b0);
      const unsigned p1 = gd_plane_pixel<kNarrow>(p, center, yslope, colormap, y0 + b1);
      gd_sts8(dst + (y0 + b0) * GD_SW, p0);
      gd_sts8(dst + (y0 + b1) * GD_SW, p1);
    }
  }
}

__device__ __noinline__ void gd_mark_plane(const GdScene &sc_, const GdView &v_, const GdShared &sh_, int x, int ya, int yb,
                              int sector, bool isFloor, unsigned *owned, const unsigned *filled) {
  const GdScene &sc = *gd_as_shared(&sc_);
  const GdView &v = *gd_as_shared(&v_);
  const GdShared &sh = *gd_as_shared(&sh_);
  if (ya >= yb) return;
  const int k0 = ya >> 5, k1 = (yb - 1) >> 5;
  unsigned any = 0;
#pragma unroll 1
  for (int k = k0; k <= k1; ++k) any |= gd_range_word(k, ya, yb) & ~owned[k * GD_SW];
  if (!any) return;
  GdPlaneSpan p;
  gd_plane_setup(sc, sh.planeTab, sector, isFloor, x, p);
  if (p.narrow) gd_plane_rows<true>(p, v.center, sh, x, ya, yb, owned, filled);
  else gd_plane_rows<false>(p, v.center, sh, x, ya, yb, owned, filled);
}

/* ---- two-sided middle textures (engine.py:13424-13745) -----------------------
 * Replayed after the planes: per column the nearest projected crossing of a
 * line that carries a middle texture on the viewer's side, clipped by the
 * drawseg snapshot the walk left for that column. */
__device__ __forceinline__ i64 gd_masked_iscale(i64 swall) {
  i64 s = (swall * GD_FU) >> 18;
  if (s >= 0 && s < 3) return 3;
  if (s > -3 && s < 0) return -3;
  return s;
}

template <bool kSplit>
__device__ __noinline__ void gd_masked_pass(const GdScene &sc_, const GdView &v_, const GdShared &sh_) {
  const GdScene &sc = *gd_as_shared(&sc_);
  const GdView &v = *gd_as_shared(&v_);
  const GdShared &sh = *gd_as_shared(&sh_);
  const int x = threadIdx.x;
  float rx, ry;
  gd_ray(v, x, rx, ry);
  float best = GD_INF;
  int w = -1, side = 0, texId = -1;
  bool leftEdge = false;
#pragma unroll 1
  for (int i = 0; i < sc.M; ++i) {
    const int k = GD_CHECK_INDEX(sc.maskedWalls[i], sc.W);
    const int sd = sh.walls[k].frontF ? 0 : 1;
    const int t = sc.sideTex[(k * 2 + sd) * 3];
    if (t < 0) continue;
#ifdef GD_CHECKED
    if (t >= sc.T) { atomicOr(gdCheckedStatus, GD_STATUS_BAD_INDEX); continue; }
#endif
    GdHit h = gd_hit_slow(sc, v, sh.walls, k, x, rx, ry);
    if (h.proj && h.d < best) { best = h.d; w = k; side = sd; texId = t; leftEdge = h.left; }
  }
  /* what this column drew, for the decal layer's depth test: the crossing's distance in
   * maskedDist (infinite: nothing), first row | end row << 8 in maskedInfo */
  if (!isfinite(best)) { sh.maskedDist[x] = GD_INF; return; }
  const GdWall &wv = sh.walls[w];
  const int front = gd_wsec(sc, w * 2), back = gd_wsec(sc, w * 2 + 1) < 0 ? 0 : gd_wsec(sc, w * 2 + 1);
  const int lightSector = side == 0 ? front : back;
  const float worldTop = fminf(gd_sec_ceil(sc, front), gd_sec_ceil(sc, back));
  const int4 ti = *reinterpret_cast<const int4 *>(&sc.texInfo[texId * 4]);
  const int tw = ti.x, th = ti.y, hbits = ti.w;
  const i64 owallTop = gd_rows<kSplit>(sc, v, sh, w, worldTop, x);
  const i64 owallBottom = gd_rows<kSplit>(sc, v, sh, w, worldTop - (float)th, x);
  const unsigned info = sh.maskedInfo[x];
  const bool hasSaved = (int)(info >> 16) == w;
  const i64 ceilClip = gd_max(owallTop, hasSaved ? (i64)((info >> 8) & 0xFF) : 0);
  const i64 floorClip = gd_min(owallBottom, hasSaved ? (i64)(info & 0xFF) : GD_VH);
  const float *soff = &sc.sideOff[(w * 2 + side) * 2];
  i64 hoff, vstepBase;
  gd_prep_wall(sc, wv, w, x, hoff, vstepBase);
  const i64 repeat = gd_rint(sc.wlen[w] * 65536.0f);
  if (side != 0) hoff = repeat - hoff;
  if (wv.sl > 0 && hoff < 0) hoff = 0;
  if (hoff >= repeat) hoff = repeat - 1;
  const int u = gd_pymod_width((hoff + gd_rint(soff[0] * 65536.0f)) >> 16, tw);
  const i64 vstep = vstepBase * (1LL << (14 - hbits));
  const i64 texMid = gd_rint((worldTop - v.viewZ) * 65536.0f + soff[1] * 65536.0f);
  /* R_DrawMaskedColumn: post rows from the drawseg's interpolated scale */
  const i64 sLeft = gd_clamp(wv.sl, 0, GD_SW - 1), sLast = gd_clamp(wv.sr - 1, 0, GD_SW - 1);
  i64 unused, startSwall, endSwall;
  gd_prep_wall(sc, wv, w, (int)sLeft, unused, startSwall);
  gd_prep_wall(sc, wv, w, (int)sLast, unused, endSwall);
  const i64 startScale = gd_div(1LL << 32, gd_masked_iscale(startSwall));
  const i64 endScale = gd_div(1LL << 32, gd_masked_iscale(endSwall));
  const i64 scaleStep = gd_div(endScale - startScale, gd_max(wv.sr - wv.sl, 1));
  const i64 spriteScale = startScale + gd_wmul(scaleStep, (i64)x - wv.sl);
  const i64 topScreen = v.center - (gd_wmul(texMid, spriteScale) >> 16);
  const i64 postTop = topScreen >> 16;
  const i64 postBottom = ((topScreen + gd_wmul(spriteScale, th) - GD_FU) >> 16) + 1;
  const i64 clippedTop = gd_max(postTop, ceilClip);
  i64 clippedBottom = gd_min(postBottom, floorClip);
  const i64 dcIscale = (vstepBase * GD_FU) >> 18;
  const i64 fracStart = texMid + gd_wmul(clippedTop, dcIscale) - (gd_wmul(v.center - GD_FU, dcIscale) >> 16);
  const i64 fracEnd = fracStart + gd_wmul(clippedBottom - clippedTop - 1, dcIscale);
  if (clippedTop < clippedBottom && clippedBottom < floorClip && fracEnd < (i64)th * GD_FU - dcIscale)
    clippedBottom += 1;
  if (!(hasSaved || leftEdge)) { sh.maskedDist[x] = GD_INF; return; }
  const float *wl = &sc.walls[w * 4];
  const bool horizontal = fabsf(wl[3] - wl[1]) < 1e-6f, vertical = fabsf(wl[2] - wl[0]) < 1e-6f;
  const i64 light = gd_sec_info(sc, lightSector).x + v.flashLight * 16 + (vertical ? 16 : (horizontal ? -16 : 0));
  const i64 vis = kSplit ? gd_line_vis(sc, sh.walls, sh.frags, w, side, x)
                         : wv.visL[side] + ((i64)x - wv.visSl[side]) * wv.visStep[side];
  const uint8_t *cm = sh.colormap + gd_wall_shade(light, vis) * 256;
  const uint8_t *col = sc.texAtlasCol + ((size_t)texId * sc.texW + u) * sc.texH;
  const unsigned base = (unsigned)(gd_shl(texMid, 16 - hbits) + (gd_wmul(vstep, GD_FU - v.center) >> 16));
  const unsigned step = (unsigned)vstep;
  const int rowA = (int)gd_max(clippedTop, 0), rowB = (int)gd_min(clippedBottom, GD_VH);
#pragma unroll 1
  for (int y = rowA; y < rowB; ++y)
    sh.frame[y * GD_SW + x] = cm[col[(base + (unsigned)y * step) >> (32 - hbits)]];
  sh.maskedDist[x] = rowA < rowB ? best : GD_INF;
  sh.maskedInfo[x] = (unsigned)max(rowA, 0) | ((unsigned)max(rowB, 0) << 8);
}

#define GD_FALLBACK_MAX (8 * GD_SW)

/* A column that has left the map (current sector -1) still takes part in the reference's
 * vectorised iterations: its decision is made against sector 0 with wall 0 selected at an
 * infinite distance (engine.py:11561-11588 clamp the sector index).  That decision can only
 * become a valid crossing through a projected left-edge owner: a wall of sector 0, or a
 * neighbour of wall 0 at one of its endpoints, whose ray-owned span starts at this very
 * column (engine.py:11589-11730, 11905-11990, 12005-12072), or through the rules that need
 * wall 0's projected span to end at this column (engine.py:11930-11962, 12073-12164).  Every
 * other column draws nothing, records nothing and changes nothing the frame depends on once
 * it is outside, so its walk can stop there.  This marks the columns that must go on. */
__device__ void gd_mark_afterlife_columns(const GdScene &sc, const GdShared &sh) {
  unsigned *busy = sh.ownerMask + 16;
  const int n0 = sc.secOff[1] - sc.secOff[0];
  const int nb0 = sc.nbDirect ? 0 : sc.nbOff[0], nb1 = sc.nbDirect ? 2 : sc.nbOff[1];
  const int total = n0 + (nb1 - nb0) + 1;
  for (int i = threadIdx.x; i < total; i += GD_THREADS) {
    int xl;
    if (i == total - 1) {
      const i64 sr = sh.walls[0].sr;
      xl = (sr >= 0 && sr < GD_SW) ? (int)sr : -1;
    } else {
      int w = i < n0 ? sc.secWalls[sc.secOff[0] + i]
                     : (sc.nbDirect ? sc.nbDirectTab[i - n0] : sc.nbIdx[nb0 + (i - n0)]);
      if (w < 0) continue;                            /* no neighbour at that endpoint */
      w = GD_CHECK_INDEX(w, sc.W);
      xl = sh.walls[w].isl;
    }
    if (xl >= 0 && xl < GD_SW) atomicOr(&busy[xl >> 5], 1u << (xl & 31));
  }
}

template <bool kSplit>
__device__ void gd_walk(const GdScene &sc_, const GdView &v_, const GdShared &sh_, GdEvent *events, int *eventCount,
                        const GdRowProj *rowproj, int *status, int startSector) {
  const GdScene &sc = *gd_as_shared(&sc_);
  const GdView &v = *gd_as_shared(&v_);
  const GdShared &sh = *gd_as_shared(&sh_);
  const int x = threadIdx.x;
  const int lane = x & 31;
  const unsigned quadBase = lane & ~3u;
  float rx, ry;
  gd_ray(v, x, rx, ry);
  unsigned *filled = gd_as_shared(sh.masks) + x, *owned = filled + 7 * GD_SW;
#pragma unroll
  for (int k = 0; k < 7; ++k) { filled[k * GD_SW] = 0; owned[k * GD_SW] = 0; }
  if (sc.M > 0) { sh.maskedDist[x] = GD_INF; sh.maskedInfo[x] = 0xFFFF0000u | GD_VH; }
  GdColState c;
  c.cur = startSector; c.ceilClip = 0; c.floorClip = GD_VH; c.prev = 0.0f;
  c.pendOwnerBoundary = c.pendEpBoundary = c.pendEpBridgeBoundary = c.pendPortalBridge = false;
  c.pendOwnerEpX = c.pendOwnerEpY = c.pendEpEpX = c.pendEpEpY = 0.0f;
  c.pendEpWall = c.pendEpBridgeIndex = c.pendPortalBridgeIndex = 0;
  c.pendPortalBridgeSector = -1;
  c.pendPortalBridgeExit = 0.0f;
  bool settled = false;
  const bool stopsOutside = !((sh.ownerMask[16 + (x >> 5)] >> (x & 31)) & 1u);
  int nEvents = 0;
  bool overflow = false;

  for (int iter = 0; iter < sc.S; ++iter) {
    if (__all_sync(0xffffffffu, settled)) break;
    GdIter it;
    if (!settled) {
      gd_column_decide<kSplit>(sc, v, sh.walls, sh.frags, sh.ownerMask, rowproj, sh.hitD, sh.hitA, sh.hitF, x, rx, ry, c, it);
    } else {
      it.wall = -1 - x; it.side = 0; it.tier[0] = it.tier[1] = it.tier[2] = false;
      it.ctop = it.clowtop = 0; it.cbot = it.cupbot = 0; it.vis = 0;
      it.rasterValid = false; it.valid = false; it.pskpp = false;
    }
    /* aligned four-column wallscan groups (engine.py:12694-12761) */
    bool same = true;
    bool groupValid[3];
    int groupBottom[3];
    {
      int w0 = __shfl_sync(0xffffffffu, it.wall, quadBase), s0 = __shfl_sync(0xffffffffu, it.side, quadBase);
#pragma unroll
      for (int k = 1; k < 4; ++k) {
        int wk = __shfl_sync(0xffffffffu, it.wall, quadBase + k), sk = __shfl_sync(0xffffffffu, it.side, quadBase + k);
        same = same && (wk == w0) && (sk == s0);
      }
#pragma unroll
      for (int tier = 0; tier < 3; ++tier) {
        int top = tier == 1 ? it.clowtop : it.ctop;
        int bot = tier == 2 ? it.cupbot : it.cbot;
        int topMax = -1, botMin = 1 << 20;
        bool all = true;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          topMax = max(topMax, __shfl_sync(0xffffffffu, top, quadBase + k));
          botMin = min(botMin, __shfl_sync(0xffffffffu, bot, quadBase + k));
          int tk = __shfl_sync(0xffffffffu, (int)it.tier[tier], quadBase + k);  /* never short-circuit a shuffle */
          all = all && (tk != 0);
        }
        groupValid[tier] = same && all && topMax < botMin;
        groupBottom[tier] = botMin;
      }
    }
    i64 firstVis = __shfl_sync(0xffffffffu, it.vis, quadBase);
    if (settled) continue;

    const GdColState before = c;
    const int wallIndex = it.wall, side = it.side;
    const GdWall &wv = sh.walls[wallIndex];
    GdEvent ev;
    ev.dist = it.distance; ev.wall = (short)wallIndex; ev.sector = -1;
    ev.t0a = ev.t0b = ev.t1a = ev.t1b = 0; ev.silTop = 0; ev.silBot = 255;
    ev.ceilA = ev.ceilB = ev.floorA = ev.floorB = 0; ev.pad0 = 0; ev.pad1 = 0;
    if (it.rasterValid) {
      /* visplane rows uncovered by this seg (engine.py:12637-12655) */
      int cpb = min(it.ctop, c.floorClip), fpt = max(it.cbot, c.ceilClip);
      ev.sector = (short)it.renderCurrent;
      if (it.markFloor && fpt < c.floorClip) {
        ev.floorA = (unsigned char)fpt; ev.floorB = (unsigned char)c.floorClip;
        gd_mark_plane(sc, v, sh, x, fpt, c.floorClip, it.renderCurrent, true, owned, filled);
      }
      if (it.markCeil && c.ceilClip < cpb) {
        ev.ceilA = (unsigned char)c.ceilClip; ev.ceilB = (unsigned char)cpb;
        gd_mark_plane(sc, v, sh, x, c.ceilClip, cpb, it.renderCurrent, false, owned, filled);
      }
      /* wall tiers */
      GdTierCtx t;
      gd_prep_wall(sc, wv, wallIndex, x, t.hoff, t.vstepBase);
      i64 repeat = gd_rint(sc.wlen[wallIndex] * 65536.0f);
      if (side != 0) t.hoff = repeat - t.hoff;
      if (wv.sl > 0 && t.hoff < 0) t.hoff = 0;
      if (t.hoff >= repeat) t.hoff = repeat - 1;
      const float *soff = &sc.sideOff[(wallIndex * 2 + side) * 2];
      t.tox = gd_rint(soff[0] * 65536.0f);
      t.yoff = soff[1];
      const float *wl = &sc.walls[wallIndex * 4];
      bool horizontal = fabsf(wl[3] - wl[1]) < 1e-6f, vertical = fabsf(wl[2] - wl[0]) < 1e-6f;
      t.light = gd_sec_info(sc, it.renderCurrent).x + v.flashLight * 16 + (vertical ? 16 : (horizontal ? -16 : 0));
      t.tailBottom = 0;
      if (it.oneSided) {
        if (it.ctop < it.cbot) {
          ev.t0a = (unsigned char)it.ctop; ev.t0b = (unsigned char)it.cbot;
          if (it.tex[0] >= 0) ev.pad0 |= 1;
          gd_draw_tier(sc, v, sh, x, it.ctop, it.cbot, 0, 0, it.tex[0], it.viewCeil, t, it.vis, firstVis,
                       groupValid[0], groupBottom[0], 0, 0, false, 0, filled);
        }
      } else {
        bool lowerCond = it.viewFloor < it.otherFloor, upperCond = it.viewCeil > it.otherCeil;
        int la = 0, lb = 0;
        if (lowerCond && it.clowtop < it.cbot) {
          la = it.clowtop; lb = it.cbot;
          ev.t1a = (unsigned char)la; ev.t1b = (unsigned char)lb;
          if (it.tex[1] >= 0) ev.pad0 |= 2;
          bool upperOn = upperCond && it.ctop < it.cupbot;
          gd_draw_tier(sc, v, sh, x, la, lb, 0, 0, it.tex[1], it.otherFloor, t, it.vis, firstVis, groupValid[1],
                       groupBottom[1], it.ctop, it.cupbot, upperOn && groupValid[2], groupBottom[2], filled);
        }
        if (upperCond && it.ctop < it.cupbot) {
          ev.t0a = (unsigned char)it.ctop; ev.t0b = (unsigned char)it.cupbot;
          if (it.tex[2] >= 0) ev.pad0 |= 1;
          gd_draw_tier(sc, v, sh, x, it.ctop, it.cupbot, la, lb, it.tex[2], it.otherCeil, t, it.vis, firstVis,
                       groupValid[2], groupBottom[2], 0, 0, false, 0, filled);
        }
      }
    }
    /* clip updates (engine.py:12885-12913) */
    bool hasUpper = it.tex[2] >= 0, hasLower = it.tex[1] >= 0;
    bool drawsUpper = (it.viewCeil > it.otherCeil) && hasUpper;
    bool drawsLower = (it.viewFloor < it.otherFloor) && hasLower;
    if (it.rasterValid && !it.oneSided && (drawsUpper || it.markCeil)) c.ceilClip = drawsUpper ? it.cupbot : it.ctop;
    if (it.rasterValid && !it.oneSided && (drawsLower || it.markFloor)) c.floorClip = drawsLower ? it.clowtop : it.cbot;
    /* masked drawseg snapshot (engine.py:12914-12939) */
    if (sc.M > 0 && it.rasterValid && !it.oneSided && it.tex[0] >= 0 && it.distance < sh.maskedDist[x]) {
      sh.maskedDist[x] = it.distance;
      sh.maskedInfo[x] = ((unsigned)wallIndex << 16) | ((unsigned)c.ceilClip << 8) | (unsigned)c.floorClip;
    }
    /* sprite silhouettes (engine.py:12940-12964) */
    if (it.rasterValid) {
      bool masked = it.tex[0] >= 0;
      bool bottomSil = !it.oneSided && ((it.viewFloor > it.otherFloor) || (v.viewZ < it.otherFloor) || masked);
      bool topSil = !it.oneSided && ((it.viewCeil < it.otherCeil) || (v.viewZ > it.otherCeil) || masked);
      if (bottomSil) ev.silBot = (unsigned char)c.floorClip;
      if (topSil) ev.silTop = (unsigned char)c.ceilClip;
      /* a crossing that draws, marks and clips nothing leaves no trace */
      bool empty = ev.t0a == ev.t0b && ev.t1a == ev.t1b && ev.silTop == 0 && ev.silBot == 255 &&
                   ev.ceilA == ev.ceilB && ev.floorA == ev.floorB;
      if (!empty) {
        if (nEvents < GD_MAX_EVENTS) events[nEvents * GD_SW + x] = ev; else overflow = true;
        nEvents++;
      }
    }
    /* clips contributed by the portal crossed behind a projected solid
     * (engine.py:12965-13069) */
    if (it.pskpp) {
      int pIdx = it.psPathIndex;
      int pSafeOther = it.psOther < 0 ? 0 : it.psOther;
      float pOtherFloor = gd_sec_floor(sc, pSafeOther), pOtherCeil = gd_sec_ceil(sc, pSafeOther);
      int pSide = it.psFromFront ? 0 : 1;
      const int32_t *ptex = &sc.sideTex[(pIdx * 2 + pSide) * 3];
      int pTop = gd_rows<kSplit>(sc, v, sh, pIdx, it.viewCeil, x), pBottom = gd_rows<kSplit>(sc, v, sh, pIdx, it.viewFloor, x);
      int pLowerTop = gd_rows<kSplit>(sc, v, sh, pIdx, pOtherFloor, x);
      int pUpperBottom = gd_rows<kSplit>(sc, v, sh, pIdx, pOtherCeil, x);
      int pct = max(pTop, c.ceilClip), pcb = min(pBottom, c.floorClip);
      int pcub = max(min(pUpperBottom, c.floorClip), pct);
      int pclt = min(max(pLowerTop, c.ceilClip), pcb);
      int4 ri = gd_sec_info(sc, it.renderCurrent), oi = gd_sec_info(sc, pSafeOther);
      bool ld = ri.x != oi.x;
      bool pDrawsUpper = (it.viewCeil > pOtherCeil) && ptex[2] >= 0;
      bool pMarksCeil = (it.viewCeil != pOtherCeil) || ri.z != oi.z || ld;
      if (pDrawsUpper || pMarksCeil) c.ceilClip = pDrawsUpper ? pcub : pct;
      bool pDrawsLower = (it.viewFloor < pOtherFloor) && ptex[1] >= 0;
      bool pMarksFloor = (it.viewFloor != pOtherFloor) || ri.y != oi.y || ld;
      if (pDrawsLower || pMarksFloor) c.floorClip = pDrawsLower ? pclt : pcb;
      bool pMasked = ptex[0] >= 0;
      bool pBottomSil = (it.viewFloor > pOtherFloor) || (v.viewZ < pOtherFloor) || pMasked;
      bool pTopSil = (it.viewCeil < pOtherCeil) || (v.viewZ > pOtherCeil) || pMasked;
      GdEvent pe;
      pe.dist = it.psDist; pe.wall = (short)pIdx; pe.sector = -1;
      pe.t0a = pe.t0b = pe.t1a = pe.t1b = 0; pe.pad0 = 0; pe.pad1 = 0;
      pe.ceilA = pe.ceilB = pe.floorA = pe.floorB = 0;
      pe.silBot = pBottomSil ? (unsigned char)c.floorClip : 255;
      pe.silTop = pTopSil ? (unsigned char)c.ceilClip : 0;
      if (pBottomSil || pTopSil) {
        if (nEvents < GD_MAX_EVENTS) events[nEvents * GD_SW + x] = pe; else overflow = true;
        nEvents++;
      }
    }
    /* traversal update (engine.py:13242-13371) */
    float prior = c.prev;
    float np = prior;
    if (it.valid) {
      if (it.nokpp) np = it.nopDist;
      else if (it.pskpp) np = it.psDist;
      else if (it.entersShared && (it.osd < it.distance)) np = prior;
      else if (it.usesGeo) np = it.gpDist;
      else np = it.distance;
    }
    if (it.valid && it.epb) np = prior;
    if (it.valid && it.cppb) np = fmaxf(it.distance, c.pendPortalBridgeExit);
    c.prev = np;
    if (it.startsOwner) { c.pendOwnerEpX = it.selEpX; c.pendOwnerEpY = it.selEpY; }
    c.pendOwnerBoundary = it.startsOwner || (c.pendOwnerBoundary && it.continuesOwner);
    if (it.endpointOnly) { c.pendEpEpX = it.epEpX; c.pendEpEpY = it.epEpY; c.pendEpWall = wallIndex; }
    c.pendEpBoundary = it.endpointOnly;
    if (it.pendEpHasFwd) c.pendEpBridgeIndex = it.epFwdIdx;
    c.pendEpBridgeBoundary = it.pendEpHasFwd;
    int next;
    if (it.nokpp) next = it.nopOther;
    else if (it.pskpp) next = it.psOther;
    else if (it.usesGeo) next = it.gpOther;
    else if (it.valid && !it.oneSided && (it.geometric || it.entersOther || it.entersShared)) next = it.otherSector;
    else if (it.endpointOnly) next = c.cur;
    else next = -1;
    if (it.epb) next = it.otherSector;
    if (it.cppb) next = c.pendPortalBridgeSector;
    if (it.epb) {
      c.pendPortalBridgeIndex = it.ppbIdx;
      c.pendPortalBridgeSector = it.gpOther;
      c.pendPortalBridgeExit = it.gpDist;
    }
    c.pendPortalBridge = it.epb;
    c.cur = next;
    /* A column that has left the map repeats the same decision on the same
     * state forever; once an iteration changes nothing and draws nothing it can
     * stop. */
    if (before.cur < 0 && !it.rasterValid && !it.pskpp && gd_state_equal(before, c)) settled = true;
    if (c.cur < 0 && stopsOutside) settled = true;
  }
  eventCount[x] = nEvents < GD_MAX_EVENTS ? nEvents : GD_MAX_EVENTS;
  if (overflow) atomicOr(status, GD_STATUS_EVENT_OVERFLOW);

}

#endif
