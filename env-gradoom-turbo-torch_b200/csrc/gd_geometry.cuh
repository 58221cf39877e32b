/* View setup, wall projection, per-(column, wall) ray tests, static topology predicates, ray-owned spans, blocking rays.
 * Part of gd_render.cu (one translation unit); not meant to be included elsewhere. */
#ifndef GD_GEOMETRY_CUH
#define GD_GEOMETRY_CUH

/* ---- view (engine.py:10648-10670, 10596-10601, 14949-14967) ------------- */
__device__ void gd_view_setup(const GdScene &sc, const int32_t *lane, GdView &v) {
  v.x = __int_as_float(lane[GD_L_X]);
  v.y = __int_as_float(lane[GD_L_Y]);
  v.angle = __int_as_float(lane[GD_L_ANGLE]);
  v.viewZ = __int_as_float(lane[GD_L_VIEW_Z]);
  v.vx = lane[GD_L_X_FIXED];
  v.vy = lane[GD_L_Y_FIXED];
  i64 bam = (i64)(uint32_t)lane[GD_L_ANGLE_BAM];
  v.pitchBam = lane[GD_L_PITCH_BAM];
  int fine = (int)((bam >> 19) & 8191);
  v.vsin = sc.fineSine[fine];
  v.vcos = sc.fineSine[(fine + 2048) & 8191];
  v.fsin = (float)v.vsin / 65536.0f;
  v.fcos = (float)v.vcos / 65536.0f;
  i64 ti = gd_clamp((GD_ANG90 - v.pitchBam) >> 19, 0, 4095);
  v.center = 104 * GD_FU + ((GD_FOCAL_Y * (i64)sc.fineTan[ti]) >> 16);
  v.upperClip = gd_div((-v.center) * GD_FU, GD_FOCAL_Y);
  v.lowerClip = gd_div((GD_VH * GD_FU - v.center) * GD_FU, GD_FOCAL_Y);
  int weapon = (int)gd_clamp(lane[GD_L_WEAPON], 0, 7);
  int cooldown = (int)gd_clamp(lane[GD_L_WPN_COOLDOWN], 0, sc.wpnTics - 1);
  int parity = (int)gd_pymod(lane[GD_L_WPN_FIRE_COUNT], 2);
  if (weapon == 1 && cooldown == 0) parity = (int)gd_pymod(gd_max(lane[GD_L_WPN_READY_TICS] - 1, 0) / 4, 2);
  v.flashLight = sc.wpnFlashLights[(weapon * 2 + parity) * sc.wpnTics + cooldown];
}

__device__ __forceinline__ void gd_ray(const GdView &v, int x, float &rx, float &ry) {
  float c = ((float)x - 160.0f) / 160.0f;
  rx = v.fcos + v.fsin * c;
  ry = v.fsin - v.fcos * c;
}

/* FWallCoords (engine.py:10791-10869) */
__device__ void gd_fwall_coords(i64 tx1, i64 ty1, i64 tx2, i64 ty2, i64 &sl, i64 &sr, i64 &dl, i64 &dr) {
  const i64 cf = 160 * GD_FU;
  i64 sty1 = ty1 == 0 ? 1 : ty1, sty2 = ty2 == 0 ? 1 : ty2;
  i64 lp = (cf + gd_div(tx1 * cf, sty1)) >> 16;
  lp += (tx1 >= 0);
  if (tx1 >= 0) lp = gd_min(lp, GD_SW);
  i64 rp = (cf + gd_div(tx2 * cf, sty2)) >> 16;
  rp += (tx2 >= 0);
  if (tx2 >= 0) rp = gd_min(rp, GD_SW);
  i64 lden = tx1 - tx2 - ty2 + ty1, rden = ty2 - ty1 - tx2 + tx1;
  i64 slden = lden == 0 ? 1 : lden, srden = rden == 0 ? 1 : rden;
  bool lin = tx1 >= -ty1, rin = tx2 <= ty2;
  i64 screenL = lin ? lp : 0, screenR = rin ? rp : GD_SW;
  i64 depthL = lin ? ty1 : ty1 + gd_div((ty2 - ty1) * (tx1 + ty1), slden);
  i64 depthR = rin ? ty2 : ty1 + gd_div((ty2 - ty1) * (tx1 - ty1), srden);
  bool invL = (lin ? ((tx1 > ty1) || (ty1 == 0)) : ((tx2 < -ty2) || (lden == 0))) || (depthL < 32);
  bool invR = (rin ? ((tx2 < -ty2) || (ty2 == 0)) : ((tx1 > ty1) || (rden == 0))) || (depthR < 32);
  bool inv = invL || invR || (screenR <= screenL);
  if (inv) screenR = screenL;
  sl = screenL; sr = screenR; dl = depthL; dr = depthR;
}

/* wallscan light for one endpoint order (engine.py:11217-11291) */
__device__ void gd_wall_visibility(i64 tx1, i64 ty1, i64 tx2, i64 ty2, i64 &visL, i64 &visStep, i64 &visSl) {
  const i64 cf = 160 * GD_FU;
  i64 sty1 = ty1 == 0 ? 1 : ty1, sty2 = ty2 == 0 ? 1 : ty2;
  i64 lp = ((cf + gd_div(tx1 * cf, sty1)) >> 16) + (tx1 >= 0);
  i64 rp = ((cf + gd_div(tx2 * cf, sty2)) >> 16) + (tx2 >= 0);
  i64 lden = tx1 - tx2 - ty2 + ty1, rden = ty2 - ty1 - tx2 + tx1;
  i64 slden = lden == 0 ? 1 : lden, srden = rden == 0 ? 1 : rden;
  bool lin = tx1 >= -ty1, rin = tx2 <= ty2;
  i64 wsl = lin ? lp : 0, wsr = rin ? rp : GD_SW;
  i64 wdl = lin ? ty1 : ty1 + gd_div((ty2 - ty1) * (tx1 + ty1), slden);
  i64 wdr = rin ? ty2 : ty1 + gd_div((ty2 - ty1) * (tx1 - ty1), srden);
  i64 ll = gd_div(GD_WALL_VIS << 12, gd_max(wdl, 1));
  i64 lr = gd_div(GD_WALL_VIS << 12, gd_max(wdr, 1));
  visStep = gd_div(lr - ll, gd_max(wsr - wsl, 1));
  visL = ll;
  visSl = wsl;
}

/* View coordinates, FWallCoords and wallscan light of a segment given by its 16.16 endpoints
 * (engine.py:10747-10869, 11207-11302). */
__device__ __noinline__ void gd_project_fixed(const GdView &v, const i64 fx[2], const i64 fy[2], GdWall &out) {
  i64 tx[2], ty[2];
#pragma unroll
  for (int e = 0; e < 2; ++e) {
    i64 rx = fx[e] - v.vx, ry = fy[e] - v.vy;
    tx[e] = (rx * v.vsin - ry * v.vcos) >> 20;
    ty[e] = (rx * v.vcos + ry * v.vsin) >> 20;
    out.tx[e] = (int)tx[e];
    out.ty[e] = (int)ty[e];
  }
  i64 wvx = fx[1] - fx[0], wvy = fy[1] - fy[0];
  i64 fsx = v.vx - fx[0], fsy = v.vy - fy[0];
  bool ff = (wvx * fsy - wvy * fsx) < 0;
  int a = ff ? 0 : 1, b = ff ? 1 : 0;
  i64 sl, sr, dl, dr;
  gd_fwall_coords(tx[a], ty[a], tx[b], ty[b], sl, sr, dl, dr);
  out.sl = sl; out.sr = sr; out.dl = dl; out.dr = dr;
  gd_wall_visibility(tx[0], ty[0], tx[1], ty[1], out.visL[0], out.visStep[0], out.visSl[0]);
  gd_wall_visibility(tx[1], ty[1], tx[0], ty[0], out.visL[1], out.visStep[1], out.visSl[1]);
}

/* Project wall w of the map for this lane (engine.py:10747-10869, 11207-11302,
 * 11359-11427).  The ray-owned span is completed by gd_wall_span below. */
__device__ __forceinline__ void gd_project_wall(const GdScene &sc, const GdView &v, int w, GdWall &out) {
  const float *wl = &sc.walls[w * 4];
  const i64 fx[2] = {gd_rint(wl[0] * 65536.0f), gd_rint(wl[2] * 65536.0f)};
  const i64 fy[2] = {gd_rint(wl[1] * 65536.0f), gd_rint(wl[3] * 65536.0f)};
  gd_project_fixed(v, fx, fy, out);
  out.oneSided = gd_wsec(sc, w * 2 + 1) < 0;
  float sx = wl[0], sy = wl[1];
  float segx = wl[2] - sx, segy = wl[3] - sy;
  float vfsx = v.x - sx, vfsy = v.y - sy;
  out.frontF = (segx * vfsy - segy * vfsx) < 0;
}

/* One piece of a line a node builder split (engine.py:11478-11500): projected like a line, from its
 * own fixed-point endpoints.  Only its FWallCoords and its wallscan light are ever read. */
__device__ __forceinline__ void gd_project_fragment(const GdScene &sc, const GdView &v, int f, GdWall &out) {
  const int4 q = *reinterpret_cast<const int4 *>(&sc.fragFixed[f * 4]);
  const i64 fx[2] = {q.x, q.z}, fy[2] = {q.y, q.w};
  gd_project_fixed(v, fx, fy, out);
  out.oneSided = 0; out.frontF = 0; out.hasColumns = 0; out.isl = 0; out.isr = 0; out.pad = 0;
}

/* Column-ray test of wall w at column x (engine.py:11317-11331).  Returns the
 * raw distance / along and the geometric-hit flag; span validity is applied by
 * gd_hit. */
__device__ __forceinline__ void gd_ray_test(const GdScene &sc, const GdView &v, int w, float rx, float ry,
                                            float &distance, float &along, bool &geo, bool &positive) {
  const float4 wl = *reinterpret_cast<const float4 *>(&sc.walls[w * 4]);
  float sx = wl.x, sy = wl.y;
  float segx = wl.z - sx, segy = wl.w - sy;
  float offx = sx - v.x, offy = sy - v.y;
  float den = rx * segy - ry * segx;
  bool small = fabsf(den) < 1e-6f;
  float safe = small ? 1.0f : den;
  distance = (offx * segy - offy * segx) / safe;
  along = (offx * ry - offy * rx) / safe;
  positive = !small && distance > 0;
  geo = positive && along >= 0 && along <= 1;
}

/* Same test without the divisions, for the span sweep: the comparisons of the
 * rounded quotients with 0 and 1 depend only on signs and magnitudes. */
__device__ __forceinline__ bool gd_ray_geo(const float4 wl, const GdView &v, float rx, float ry) {
  float sx = wl.x, sy = wl.y;
  float segx = wl.z - sx, segy = wl.w - sy;
  float offx = sx - v.x, offy = sy - v.y;
  float den = rx * segy - ry * segx;
  bool small = fabsf(den) < 1e-6f;
  float safe = small ? 1.0f : den;
  float dn = offx * segy - offy * segx;
  float an = offx * ry - offy * rx;
  /* dn / safe > 0: both are differences of products of map-scale numbers, so a
   * nonzero dn is far too large for the quotient to underflow to zero */
  bool positive = (dn != 0.0f) && ((dn < 0) == (safe < 0));
  bool alongOk = (an == 0.0f) || (((an < 0) == (safe < 0)) && fabsf(an) <= fabsf(safe));
  return !small && positive && alongOk;
}

/* ---- per (column, wall) hit -------------------------------------------- */
struct GdHit {
  float d;       /* ray distance, +inf when the wall does not count here */
  float along;   /* clamped to [0,1] */
  bool geo, proj, left;
};

/* engine.py:11440-11459 */
__device__ __forceinline__ GdHit gd_hit(const GdScene &sc, const GdView &v, const GdWall *walls, int w, int x,
                                        float rx, float ry) {
  GdHit h;
  float distance, along;
  bool geo, positive;
  w = GD_CHECK_INDEX(w, sc.W);
  gd_ray_test(sc, v, w, rx, ry, distance, along, geo, positive);
  const GdWall &wv = walls[w];
  bool screenValid = wv.hasColumns && x >= wv.isl && x < wv.isr;
  bool pv = positive && screenValid;
  bool valid = wv.oneSided ? (pv && wv.frontF) : (geo || pv);
  h.d = valid ? distance : GD_INF;
  float ac = along;
  if (!(ac >= 0.0f)) ac = (ac != ac) ? ac : 0.0f;
  if (ac > 1.0f) ac = 1.0f;
  h.along = ac;
  h.geo = geo;
  h.proj = pv;
  h.left = (x == wv.isl);
  return h;
}

__device__ __noinline__ GdHit gd_hit_slow(const GdScene &sc_, const GdView &v_, const GdWall *walls, int w, int x,
                                          float rx, float ry) {
  const GdScene &sc = *gd_as_shared(&sc_);
  const GdView &v = *gd_as_shared(&v_);
  return gd_hit(sc, v, walls, w, x, rx, ry);
}

__device__ __forceinline__ float gd_tol(float d) { return fmaxf(fabsf(d) / 128.0f, 4.0f); }

/* Endpoint owner of wall w at column x (engine.py:11589-11730). */
__device__ __noinline__ void gd_endpoint_owner(const GdScene &sc_, const GdView &v_, const GdWall *walls, int w, int x, float rx,
                                  float ry, const GdHit &hw, int &ownerIdx, float &ownerDist) {
  const GdScene &sc = *gd_as_shared(&sc_);
  const GdView &v = *gd_as_shared(&v_);
  const GdWall &wv = walls[w];
  float d = hw.d;
  float tol = gd_tol(d);
  bool subpixel = (wv.sr - wv.sl <= 1) && !wv.oneSided;
  bool usesStart = hw.along <= 0.5f;
  int oi = w;
  float od = d;
  bool ownerValid = false;
  if (sc.nbDirect) {
    const int32_t *nd = &sc.nbDirectTab[w * 4];
    int sIdx = nd[0] >= 0 ? GD_CHECK_INDEX(nd[0], sc.W) : w, eIdx = nd[1] >= 0 ? GD_CHECK_INDEX(nd[1], sc.W) : w;
    bool hasS = nd[0] >= 0, hasE = nd[1] >= 0;
    int rIdx = usesStart ? sIdx : eIdx, rSlot = usesStart ? nd[2] : nd[3];
    bool rHas = usesStart ? hasS : hasE;
    int oIdx = usesStart ? eIdx : sIdx, oSlot = usesStart ? nd[3] : nd[2];
    bool oHas = usesStart ? hasE : hasS;
    GdHit hr = (rIdx == w) ? hw : gd_hit(sc, v, walls, rIdx, x, rx, ry);
    GdHit ho = (oIdx == w) ? hw : gd_hit(sc, v, walls, oIdx, x, rx, ry);
    bool rOwns = rHas && hr.proj && hr.left;
    bool oOwns = subpixel && oHas && ho.proj && ho.left && (fabsf(ho.d - d) <= tol);
    bool useO = oOwns && (!rOwns || ho.d < hr.d || (ho.d == hr.d && oSlot < rSlot));
    oi = useO ? oIdx : rIdx;
    od = useO ? ho.d : hr.d;
    ownerValid = rOwns || oOwns;
  } else {
    float best = GD_INF;
    int bestSlot = 0;
    int n0 = sc.nbOff[w], n1 = sc.nbOff[w + 1];
#pragma unroll 1
    for (int k = n0; k < n1; ++k) {
      int nb = GD_CHECK_INDEX(sc.nbIdx[k], sc.W), fl = sc.nbFlags[k];
      GdHit hn = gd_hit(sc, v, walls, nb, x, rx, ry);
      bool rayNb = usesStart ? (fl & 1) : ((fl >> 1) & 1);
      bool sel = rayNb || (subpixel && (fabsf(hn.d - d) <= tol));
      float cand = (hn.proj && hn.left && sel) ? hn.d : GD_INF;
      if (cand < best) { best = cand; bestSlot = k - n0; }
    }
    od = best;
    oi = (n1 > n0) ? GD_CHECK_INDEX(sc.nbIdx[n0 + bestSlot], sc.W) : w;
    ownerValid = isfinite(best);
  }
  bool has = !hw.proj && ownerValid;
  ownerIdx = has ? oi : w;
  ownerDist = has ? od : d;
}

/* PrepWall for one (column, wall) (engine.py:10672-10739). */
__device__ __noinline__ void gd_prep_wall(const GdScene &sc_, const GdWall &wv, int w, int x, i64 &hoff, i64 &vstep) {
  const GdScene &sc = *gd_as_shared(&sc_);
  i64 tx1 = wv.tx[0], tx2 = wv.tx[1], ty1 = wv.ty[0], ty2 = wv.ty[1];
  double uozOrigin = (double)((float)tx1 * 160.0f);
  double uozStep = (double)(-(float)ty1);
  double invzOrigin = (double)((float)(tx1 - tx2) * 160.0f);
  float invzStepF = (float)(ty2 - ty1);
  double invzStep = (double)invzStepF;
  double col = (double)x - 160.0;
  double top = uozOrigin + uozStep * col;
  double bottom = invzOrigin + invzStep * col;
  double safeBottom = bottom == 0 ? 1.0 : bottom;
  double fraction = top / safeBottom;
  i64 repeat = gd_rint(sc.wlen[w] * 65536.0f);
  hoff = (i64)floor(fraction * (double)repeat + 0.5);
  const double wms = (320 * 200.0 / 320.0 / 240) * 64.0 / (320 / 2.0);
  double depthScale = (double)(invzStepF * (float)wms);
  double depthOrigin = (double)((-(float)uozStep) * (float)wms);
  vstep = (i64)floor(fraction * depthScale + depthOrigin + 0.5);
}

/* OWallMost row projection (engine.py:12294-12605), one fragment per wall. */
__device__ __noinline__ int gd_project_rows(const GdView &v_, const GdWall &wv, float worldZ, int x) {
  const GdView &v = *gd_as_shared(&v_);
  i64 wsl = wv.sl, wsr = wv.sr;
  i64 wdl = gd_max(wv.dl, 1), wdr = gd_max(wv.dr, 1);
  bool owns = (wsr > wsl) && x >= wsl && x < wsr;
  i64 relZ = gd_rint((worldZ - v.viewZ) * 65536.0f);
  i64 pz = -(relZ >> 4);
  i64 center = v.center;
  i64 num = pz * GD_FOCAL_Y;
  if (!owns) {
    i64 ospan = gd_max(wsr - wsl, 1);
    i64 opl = gd_div(num, wdl), opr = gd_div(num, wdr);
    i64 ostep = gd_div(opr - opl, ospan);
    return (int)gd_clamp((center + opl + (x - wsl) * ostep) >> 16, 0, GD_VH);
  }
  i64 sl = wsl, sr = wsr, dl = wdl, dr = wdr;
  i64 upperClip = v.upperClip, lowerClip = v.lowerClip;
  i64 ul = (upperClip * dl) >> 16, ur = (upperClip * dr) >> 16;
  i64 ll = (lowerClip * dl) >> 16, lr = (lowerClip * dr) >> 16;
  bool aboveL = pz < ul, aboveR = pz < ur, belowL = pz > ll, belowR = pz > lr;
  bool entAbove = aboveL && aboveR, entBelow = belowL && belowR;
  i64 cl = sl, cr = sr, cdl = dl, cdr = dr;
  bool outTop = false, outBottom = false;
  bool crossesTop = aboveL != aboveR;
  if (crossesTop) {
    i64 sud = (ur != ul) ? (ur - ul) : 1;
    i64 tf = gd_div(gd_shl(pz - ul, 30), sud);
    i64 td = dl + (((dr - dl) * tf) >> 30);
    i64 tc = sl + gd_div(((dr * tf) >> 30) * (sr - sl), gd_max(td, 1));
    if (aboveR && (sl <= tc)) { cr = tc; cdr = td; }
    outTop |= aboveR && (sr > tc) && (x >= tc) && (x < sr);
    if (aboveL && (tc <= sr)) { cl = tc; cdl = td; }
    outTop |= aboveL && (tc > sl) && (x >= sl) && (x < tc);
  }
  bool crossesBottom = belowL != belowR;
  if (crossesBottom) {
    i64 sld = (lr != ll) ? (lr - ll) : 1;
    i64 bf = gd_div(gd_shl(pz - ll, 30), sld);
    i64 bd = dl + (((dr - dl) * bf) >> 30);
    i64 bc = sl + gd_div(((dr * bf) >> 30) * (sr - sl), gd_max(bd, 1));
    if (belowR && (sl <= bc)) { cr = bc; cdr = bd; }
    outBottom |= belowR && (sr > bc) && (x >= bc) && (x < sr);
    if (belowL && (bc <= sr)) { cl = bc; cdl = bd; }
    outBottom |= belowL && (bc > sl) && (x >= sl) && (x < bc);
  }
  bool collapsed = (cr == cl) && (x == cl) && !(entAbove || entBelow);
  if (entAbove || (outTop && !collapsed)) return 0;
  if (entBelow || (outBottom && !collapsed)) return GD_VH;
  i64 pl = gd_div(num, gd_max(cdl, 1)), pr = gd_div(num, gd_max(cdr, 1));
  i64 span = gd_max(cr - cl, 1);
  i64 pstep = gd_div(pr - pl, span);
  return (int)gd_clamp((center + pl + (x - cl) * pstep) >> 16, 0, GD_VH);
}

/* The unclipped whole-line projection: what a column of a split line falls back to when none of
 * the line's fragments owns it (engine.py:12393-12410, 12596-12604). */
__device__ __noinline__ int gd_project_rows_whole(const GdView &v, const GdWall &wv, float worldZ, int x) {
  const i64 wdl = gd_max(wv.dl, 1), wdr = gd_max(wv.dr, 1);
  const i64 relZ = gd_rint((worldZ - v.viewZ) * 65536.0f);
  const i64 num = -(relZ >> 4) * GD_FOCAL_Y;
  const i64 opl = gd_div(num, wdl), opr = gd_div(num, wdr);
  const i64 ostep = gd_div(opr - opl, gd_max(wv.sr - wv.sl, 1));
  return (int)gd_clamp((v.center + opl + (x - wv.sl) * ostep) >> 16, 0, GD_VH);
}

/* Is line w split, and if so which of its fragments owns column x: the first whose half-open
 * span holds it (engine.py:12310-12376, 11511-11545), or null. */
__device__ __forceinline__ bool gd_line_is_split(const GdScene &sc, int w) {
  return sc.F > 0 && sc.fragOff[w + 1] > sc.fragOff[w];
}
__device__ __noinline__ const GdWall *gd_fragment_at(const GdScene &sc, const GdWall *frags, int w, int x) {
#pragma unroll 1
  for (int f = sc.fragOff[w]; f < sc.fragOff[w + 1]; ++f) {
    const GdWall &q = frags[f];
    if (q.sr > q.sl && x >= q.sl && x < q.sr) return &q;
  }
  return nullptr;
}
/* Row projection and wallscan light of line w at column x, fragments considered. */
__device__ __noinline__ int gd_line_rows(const GdScene &sc, const GdView &v, const GdWall *walls, const GdWall *frags, int w,
                                         float worldZ, int x) {
  if (!gd_line_is_split(sc, w)) return gd_project_rows(v, walls[w], worldZ, x);
  const GdWall *q = gd_fragment_at(sc, frags, w, x);
  return q ? gd_project_rows(v, *q, worldZ, x) : gd_project_rows_whole(v, walls[w], worldZ, x);
}
__device__ __forceinline__ i64 gd_line_vis(const GdScene &sc, const GdWall *walls, const GdWall *frags, int w, int side, int x) {
  const GdWall *q = &walls[w];
  if (gd_line_is_split(sc, w)) {
    const GdWall *f = gd_fragment_at(sc, frags, w, x);
    if (f) q = f;
  }
  return q->visL[side] + ((i64)x - q->visSl[side]) * q->visStep[side];
}

/* Column-independent part of gd_project_rows for one (wall, height). */
__device__ __noinline__ void gd_rowproj_setup(const GdView &v_, const GdWall &wv, float worldZ, GdRowProj &o) {
  const GdView &v = *gd_as_shared(&v_);
  i64 wsl = wv.sl, wsr = wv.sr;
  i64 wdl = gd_max(wv.dl, 1), wdr = gd_max(wv.dr, 1);
  i64 relZ = gd_rint((worldZ - v.viewZ) * 65536.0f);
  i64 pz = -(relZ >> 4);
  i64 num = pz * GD_FOCAL_Y;
  {
    i64 ospan = gd_max(wsr - wsl, 1);
    i64 opl = gd_div(num, wdl), opr = gd_div(num, wdr);
    o.opl = opl;
    o.ostep = gd_div(opr - opl, ospan);
  }
  i64 sl = wsl, sr = wsr, dl = wdl, dr = wdr;
  i64 upperClip = v.upperClip, lowerClip = v.lowerClip;
  i64 ul = (upperClip * dl) >> 16, ur = (upperClip * dr) >> 16;
  i64 ll = (lowerClip * dl) >> 16, lr = (lowerClip * dr) >> 16;
  bool aboveL = pz < ul, aboveR = pz < ur, belowL = pz > ll, belowR = pz > lr;
  bool entAbove = aboveL && aboveR, entBelow = belowL && belowR;
  i64 cl = sl, cr = sr, cdl = dl, cdr = dr;
  i64 topA = 0, topB = 0, botA = 0, botB = 0;
  if (aboveL != aboveR) {
    i64 sud = (ur != ul) ? (ur - ul) : 1;
    i64 tf = gd_div(gd_shl(pz - ul, 30), sud);
    i64 td = dl + (((dr - dl) * tf) >> 30);
    i64 tc = sl + gd_div(((dr * tf) >> 30) * (sr - sl), gd_max(td, 1));
    if (aboveR && (sl <= tc)) { cr = tc; cdr = td; }
    if (aboveR && (sr > tc)) { topA = tc; topB = sr; }
    if (aboveL && (tc <= sr)) { cl = tc; cdl = td; }
    if (aboveL && (tc > sl)) { topA = sl; topB = tc; }
  }
  if (belowL != belowR) {
    i64 sld = (lr != ll) ? (lr - ll) : 1;
    i64 bf = gd_div(gd_shl(pz - ll, 30), sld);
    i64 bd = dl + (((dr - dl) * bf) >> 30);
    i64 bc = sl + gd_div(((dr * bf) >> 30) * (sr - sl), gd_max(bd, 1));
    if (belowR && (sl <= bc)) { cr = bc; cdr = bd; }
    if (belowR && (sr > bc)) { botA = bc; botB = sr; }
    if (belowL && (bc <= sr)) { cl = bc; cdl = bd; }
    if (belowL && (bc > sl)) { botA = sl; botB = bc; }
  }
  bool collapsed = (cr == cl) && !(entAbove || entBelow);
  o.collapsedX = (short)((collapsed && cl >= 0 && cl < GD_SW) ? cl : -1);
  o.entAbove = entAbove; o.entBelow = entBelow;
  o.topA = (short)gd_clamp(topA, -1, GD_SW + 1); o.topB = (short)gd_clamp(topB, -1, GD_SW + 1);
  o.botA = (short)gd_clamp(botA, -1, GD_SW + 1); o.botB = (short)gd_clamp(botB, -1, GD_SW + 1);
  i64 pl = gd_div(num, gd_max(cdl, 1)), pr = gd_div(num, gd_max(cdr, 1));
  o.pl = pl;
  o.pstep = gd_div(pr - pl, gd_max(cr - cl, 1));
  o.cl = cl;
  o.pad = 0;
}

__device__ __forceinline__ int gd_rowproj_eval(const GdView &v, const GdWall &wv, const GdRowProj &o, int x) {
  bool owns = (wv.sr > wv.sl) && x >= wv.sl && x < wv.sr;
  if (!owns) return (int)gd_clamp((v.center + o.opl + (x - wv.sl) * o.ostep) >> 16, 0, GD_VH);
  bool collapsed = x == o.collapsedX;
  bool outTop = x >= o.topA && x < o.topB, outBottom = x >= o.botA && x < o.botB;
  if (o.entAbove || (outTop && !collapsed)) return 0;
  if (o.entBelow || (outBottom && !collapsed)) return GD_VH;
  return (int)gd_clamp((v.center + o.pl + (x - o.cl) * o.pstep) >> 16, 0, GD_VH);
}

__device__ __forceinline__ int gd_wall_shade(i64 light, i64 vis) {
  i64 base = 64 * GD_FU - (light + 12) * (GD_FU / 4);
  return (int)gd_clamp((base - gd_min(vis, 24 * GD_FU)) >> 16, 0, 31);
}

/* ---- static topology predicates (engine.py:399-484, 1596-1612) ---------- */
__device__ __forceinline__ int gd_secidx(const GdScene &sc, int s) { return GD_CHECK_SECTOR(s < 0 ? s + sc.S : s, sc.S); }
__device__ __forceinline__ float gd_sec_floor(const GdScene &sc, int s) { return sc.secF[gd_secidx(sc, s) * 2]; }
__device__ __forceinline__ float gd_sec_ceil(const GdScene &sc, int s) { return sc.secF[gd_secidx(sc, s) * 2 + 1]; }
__device__ __forceinline__ int4 gd_sec_info(const GdScene &sc, int s) {
  return *reinterpret_cast<const int4 *>(&sc.secI[gd_secidx(sc, s) * 4]);
}

__device__ __forceinline__ bool gd_same_pair(const GdScene &sc, int a, int b) {
  int a0 = gd_wsec(sc, a * 2), a1 = gd_wsec(sc, a * 2 + 1), b0 = gd_wsec(sc, b * 2), b1 = gd_wsec(sc, b * 2 + 1);
  return (a0 == b0 && a1 == b1) || (a0 == b1 && a1 == b0);
}
__device__ __forceinline__ bool gd_shares_endpoint(const GdScene &sc, int a, int b) {
  int a0 = sc.wvtx[a * 2], a1 = sc.wvtx[a * 2 + 1], b0 = sc.wvtx[b * 2], b1 = sc.wvtx[b * 2 + 1];
  return a0 == b0 || a0 == b1 || a1 == b0 || a1 == b1;
}
__device__ __noinline__ bool gd_opposing_pair(const GdScene &sc_, int a, int b) {
  const GdScene &sc = *gd_as_shared(&sc_);
  if (!gd_same_pair(sc, a, b)) return false;
  if (gd_wsec(sc, a * 2 + 1) < 0 || gd_wsec(sc, b * 2 + 1) < 0) return false;
  if (gd_shares_endpoint(sc, a, b)) return false;
  const float *A = &sc.walls[a * 4], *B = &sc.walls[b * 4];
  float adx = A[2] - A[0], ady = A[3] - A[1], bdx = B[2] - B[0], bdy = B[3] - B[1];
  float dot = adx * bdx + ady * bdy;
  float cross = adx * bdy - ady * bdx;
  return dot < 0 && fabsf(cross) < 1e-6f;
}
__device__ __forceinline__ bool gd_two_distinct(const GdScene &sc, int w) {
  return gd_wsec(sc, w * 2 + 1) >= 0 && gd_wsec(sc, w * 2) != gd_wsec(sc, w * 2 + 1);
}
__device__ bool gd_bridge_pair_of(const GdScene &sc, int a, int b, int &p0, int &p1) {
  int a0 = gd_wsec(sc, a * 2), a1 = gd_wsec(sc, a * 2 + 1), b0 = gd_wsec(sc, b * 2), b1 = gd_wsec(sc, b * 2 + 1);
  int shared = 0, sv = -2;
  if (a0 == b0 || a0 == b1) { shared++; sv = a0; }
  if (a1 == b0 || a1 == b1) { shared++; sv = a1; }
  if (shared != 1) return false;
  p0 = (a0 == sv) ? a1 : a0;
  p1 = (b0 == sv) ? b1 : b0;
  return true;
}
__device__ __forceinline__ bool gd_set_equals(const GdScene &sc, int w, int p0, int p1) {
  int s0 = gd_wsec(sc, w * 2), s1 = gd_wsec(sc, w * 2 + 1);
  if (p0 == p1) return s0 == p0 && s1 == p0;
  return (s0 == p0 && s1 == p1) || (s0 == p1 && s1 == p0);
}
__device__ bool gd_unique_at_vertex(const GdScene &sc, int v, int skipA, int skipB, int p0, int p1, int &index) {
  int count = 0, found = 0;
#pragma unroll 1
  for (int k = sc.vtxOff[v]; k < sc.vtxOff[v + 1]; ++k) {
    int c = GD_CHECK_INDEX(sc.vtxWalls[k], sc.W);
    if (c == skipA || c == skipB) continue;
    if (gd_set_equals(sc, c, p0, p1)) { count++; found = c; }
  }
  index = (count == 1) ? found : 0;
  return count == 1;
}
__device__ __noinline__ bool gd_portal_bridge(const GdScene &sc_, int slot, int path, int owner, int &index) {
  const GdScene &sc = *gd_as_shared(&sc_);
  index = 0;
  if (!gd_two_distinct(sc, path) || owner == path) return false;
  int v = sc.wvtx[path * 2 + slot];
  if (sc.wvtx[owner * 2] != v && sc.wvtx[owner * 2 + 1] != v) return false;
  if (!gd_two_distinct(sc, owner)) return false;
  int p0, p1;
  if (!gd_bridge_pair_of(sc, path, owner, p0, p1)) return false;
  return gd_unique_at_vertex(sc, v, path, owner, p0, p1, index);
}
__device__ __noinline__ bool gd_sector_bridge(const GdScene &sc_, int slot, int pending, int path, int &index) {
  const GdScene &sc = *gd_as_shared(&sc_);
  index = 0;
  if (!gd_two_distinct(sc, pending) || path == pending || !gd_two_distinct(sc, path)) return false;
  int p0, p1;
  if (!gd_bridge_pair_of(sc, pending, path, p0, p1)) return false;
  return gd_unique_at_vertex(sc, sc.wvtx[pending * 2 + slot], pending, path, p0, p1, index);
}

/* ---- phase: ray-owned spans (engine.py:11333-11438) --------------------- */
/* A wall whose two endpoints lie behind the viewer, or both beyond the same
 * edge of the 90-degree frustum, is crossed by no column ray at a positive
 * distance.  The two-unit margin is four orders of magnitude above the float
 * error of these dot products at map scale, so the test only ever drops walls
 * for which the exact sweep below finds no column. */
__device__ __forceinline__ bool gd_wall_in_frustum(const float4 wl, const GdView &v) {
  float ax = wl.x - v.x, ay = wl.y - v.y, bx = wl.z - v.x, by = wl.w - v.y;
  float fa = ax * v.fcos + ay * v.fsin, fb = bx * v.fcos + by * v.fsin;      /* forward */
  float sa = ax * v.fsin - ay * v.fcos, sb = bx * v.fsin - by * v.fcos;      /* to the right */
  const float m = -2.0f;
  if (fa < m && fb < m) return false;
  if (fa + sa < m && fb + sb < m) return false;
  if (fa - sa < m && fb - sb < m) return false;
  return true;
}

__device__ void gd_wall_spans(const GdScene &sc_, const GdView &v_, const GdShared &sh_) {
  const GdScene &sc = *gd_as_shared(&sc_);
  const GdView &v = *gd_as_shared(&v_);
  const GdShared &sh = *gd_as_shared(&sh_);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  GdWall *walls = sh.walls;
  short *list = (short *)sh.hitD;           /* walls that need the sweep */
  if (threadIdx.x == 0) sh.misc[2] = 0;
  __syncthreads();
  for (int w = threadIdx.x; w < sc.W; w += GD_THREADS) {
    const float4 wl = *reinterpret_cast<const float4 *>(&sc.walls[w * 4]);
    walls[w].isl = -1;
    walls[w].isr = -1;
    if (gd_wall_in_frustum(wl, v)) list[atomicAdd(&sh.misc[2], 1)] = (short)w;
  }
  __syncthreads();
  const int n = sh.misc[2];
  float rxs[GD_SW / 32], rys[GD_SW / 32];
#pragma unroll
  for (int chunk = 0; chunk < GD_SW / 32; ++chunk) gd_ray(v, chunk * 32 + lane, rxs[chunk], rys[chunk]);
  /* first and last column whose ray crosses the wall, kept in isl / isr */
  for (int i = warp; i < n; i += GD_WARPS) {
    const int w = list[i];
    const float4 wl = *reinterpret_cast<const float4 *>(&sc.walls[w * 4]);
    int first = -1, last = -1;
#pragma unroll
    for (int chunk = 0; chunk < GD_SW / 32; ++chunk) {
      unsigned m = __ballot_sync(0xffffffffu, gd_ray_geo(wl, v, rxs[chunk], rys[chunk]));
      if (m) {
        if (first < 0) first = chunk * 32 + __ffs(m) - 1;
        last = chunk * 32 + 31 - __clz(m);
      }
    }
    if (lane == 0) { walls[w].isl = (short)first; walls[w].isr = (short)last; }
  }
  __syncthreads();
  for (int w = threadIdx.x; w < sc.W; w += GD_THREADS) {
    GdWall &wv = walls[w];
    const int first = wv.isl, last = wv.isr;
    bool hasColumns = first >= 0;
    i64 isl = hasColumns ? first : 0;
    i64 isr = hasColumns ? last + 1 : GD_SW;
    const i64 cf = 160 * GD_FU;
    i64 ecol[2];
    bool evis[2];
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      i64 ty = wv.ty[e], tx = wv.tx[e];
      i64 sty = ty == 0 ? 1 : ty;
      i64 pf = cf + gd_div(tx * cf, sty);
      ecol[e] = (pf >> 16) + (tx >= 0);
      evis[e] = ty > 0 && tx >= -ty && tx <= ty && ecol[e] >= 0 && ecol[e] <= GD_SW;
    }
    bool fff = wv.frontF;
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      bool visible = evis[e] && hasColumns;
      bool ownsLeft = fff ? (e == 0) : (e == 1);
      if (visible && ownsLeft) isl = ecol[e];
      if (visible && !ownsLeft) isr = ecol[e];
    }
    if (evis[0] && evis[1]) {
      isl = ecol[fff ? 0 : 1];
      isr = ecol[fff ? 1 : 0];
      hasColumns = isr > isl;
    }
    hasColumns = hasColumns && (wv.sr > wv.sl);
    wv.isl = (short)isl;
    wv.isr = (short)isr;
    wv.hasColumns = hasColumns;
  }
}

/* ---- phase: blocking ray cast of column x (engine.py:10534-10557) ------- */
/* Nearest one-sided wall the column ray crosses; among equal distances the
 * lowest wall index, as the reference's first-minimum over its ascending
 * blocking list.  Only walls that passed the frustum test can be crossed, and
 * the division is spent only on walls the sign test says are crossed. */
__device__ void gd_blocking_raycast(const GdScene &sc_, const GdView &v_, const GdShared &sh_, const short *list, int listed,
                                    float rx, float ry, float &wallDistance, int &blockingWall) {
  const GdScene &sc = *gd_as_shared(&sc_);
  const GdView &v = *gd_as_shared(&v_);
  const GdShared &sh = *gd_as_shared(&sh_);
  float best = GD_INF;
  int bestWall = GD_CHECK_INDEX(sc.blocking[0], sc.W);
#pragma unroll 1
  for (int i = 0; i < listed; ++i) {
    const int w = list[i];
    if (!sh.walls[w].oneSided) continue;
    const float4 wl = *reinterpret_cast<const float4 *>(&sc.walls[w * 4]);
    if (!gd_ray_geo(wl, v, rx, ry)) continue;
    float distance, along;
    bool geo, positive;
    gd_ray_test(sc, v, w, rx, ry, distance, along, geo, positive);
    float d = geo ? distance : GD_INF;
    if (d < best || (d == best && w < bestWall && isfinite(d))) { best = d; bestWall = w; }
  }
  blockingWall = bestWall;
  wallDistance = fminf(fmaxf(best, 1.0f), 4096.0f);
}

#endif
