/*
 * Fused render-to-observation kernel for sm_100a.
 *
 * One persistent CTA of 320 threads draws one environment lane at a time:
 *   1. every wall of the map is projected once per lane into shared memory
 *      (threads over walls), and its ray-owned column span is found by a warp
 *      sweeping the 320 column rays with ballots;
 *   2. thread x then walks column x front to back through the sector portals,
 *      keeping the ceiling / floor clip pair in registers, drawing wall tiers
 *      and the visplane rows they uncover straight into the palette-indexed
 *      frame held in shared memory (aligned groups of four columns exchange
 *      their tier bounds with warp shuffles);
 *   3. thread x draws the depth-sorted sprites of column x against the clip
 *      events its walk recorded;
 *   4. the weapon and, on request, the status bar are composited;
 *   5. the 320x240 frame is reduced to the 84x84 grayscale observation with the
 *      exact integer area weights and written, 16 bytes per store, into the
 *      four-frame stack; the RGB24 frame is written only when asked for.
 * Only the lane record, the thing records and the stack slot touch HBM; the
 * indexed frame never leaves the SM.  Tensor cores are unused: nothing here is
 * a contraction.
 *
 * The arithmetic restates src/gradoom/engine.py (file:line beside each
 * function) and must stay bit-identical to it; compile with -fmad=false.
 */
#include "gd_device.cuh"

#define GD_THREADS 320
#define GD_WARPS (GD_THREADS / 32)
#define GD_INF CUDART_INF_F

/* render flags */
#define GD_F_MASK_HUD 1     /* observation sees 32 black rows instead of the status bar */
#define GD_F_DRAW_HUD 2     /* composite the status bar (needed for RGB / unmasked obs) */
#define GD_F_STACK_ROLL 4   /* shift the stack by one slot and append */
#define GD_F_STACK_FILL 8   /* write all four slots of lanes whose mask byte is set */
#define GD_F_WRITE_OBS 16   /* write plain (n,84,84) observations to obsOut */

struct GdParams {
  GdScene sc;
  const int32_t *lanes;
  const gd_thing *things;
  int maxThings;
  int n;
  int flags;
  uint8_t *stack;            /* n x 4 x 84 x 84 */
  const uint8_t *resetMask;  /* n, for GD_F_STACK_FILL */
  uint8_t *obsOut;           /* n x 84 x 84, optional */
  uint8_t *indexedOut;       /* n x 240 x 320, optional */
  uint8_t *rgbOut;           /* n x 240 x 320 x 3, optional */
  uint8_t *scratch;          /* ctas x gd_scratch_per_cta(W), then the lane queue (2 words, zero between launches) */
  size_t queueOffset;
  int stageMask;             /* which scene tables each CTA copies into shared memory */
  int secWallsN, vtxWallsN, V;
  int *status;
};

#define GD_SCRATCH_EVENTS_BYTES (GD_MAX_EVENTS * GD_SW * (int)sizeof(GdEvent))
#define GD_SCRATCH_VSEC_BYTES (GD_VH * GD_SW * 2)   /* flat fallback: vertically repaired sector per pixel */
#define GD_SCRATCH_FIXED (GD_SCRATCH_EVENTS_BYTES + GD_SW * 4 + GD_SCRATCH_VSEC_BYTES)
#define GD_PLANE_ENTRY_BYTES 88          /* sizeof(GdPlaneEntry), checked below */
__host__ __device__ inline size_t gd_scratch_plane_bytes(int S) { return ((size_t)S * 2 * GD_PLANE_ENTRY_BYTES + 15) & ~(size_t)15; }
__host__ __device__ inline size_t gd_scratch_per_cta(int W, int S) {
  return (GD_SCRATCH_FIXED + gd_scratch_plane_bytes(S) + (size_t)W * 4 * sizeof(GdRowProj) + 15) & ~(size_t)15;
}

struct GdActor {
  float x, y, depth;
  i64 depthFixed, xstep, yscale, topFixed, texMid, iscale;
  int left, right;
  int sprite, w, h;
  short shade;
  signed char style;
  unsigned char alive;
};

/* ---- shared memory carve-up -------------------------------------------- */
struct GdPlaneEntry;

struct GdShared {
  GdPlaneEntry *planeTab; /* scratch: per (sector, floor/ceiling) span setup of the lane being drawn */
  uint8_t *frame;       /* 240 x 320 */
  uint8_t *colormap;    /* 32 x 256 */
  uint8_t *playpal;     /* 768 */
  unsigned *yslope;     /* 208 */
  int32_t *lane;        /* 32 */
  float *wallDistance;  /* 320 */
  short *blockingWall;  /* 320 */
  unsigned *ownerMask;  /* 10 words: boundary_has_projected_owner */
  GdWall *walls;        /* W */
  GdActor *actors;      /* maxThings */
  unsigned long long *pal64;  /* 256: R | G<<20 | B<<40 */
  uint8_t *obs;         /* 84 x 84 */
  int *misc;            /* 16 ints: start sector, fallback queue length, its unresolved rows' range, GdFlatBounds */
  unsigned *masks;      /* 14 x 320: per-column filled / plane-owned row bitmasks */
  unsigned *pal32;      /* 256: the lane's palette as r | g << 8 | b << 16, for the RGB24 output */
  float *maskedDist;    /* 320: nearest masked drawseg of the column ... */
  unsigned *maskedInfo; /* ... its wall << 16 | ceiling clip << 8 | floor clip; 0xFFFF0000 | .. = none */
  float *hitD, *hitA;   /* 8 x 320 each: per-column cache of this iteration's wall hits */
  uint8_t *hitF;        /* 8 x 320 */
};

__host__ __device__ inline size_t gd_align16(size_t v) { return (v + 15) & ~(size_t)15; }

__host__ __device__ inline size_t gd_shared_bytes(int W, int maxThings) {
  size_t b = 0;
  b += gd_align16((size_t)GD_SCREEN_H * GD_SW);
  b += gd_align16(32 * 256);
  b += gd_align16(768);
  b += gd_align16(GD_VH * 4);
  b += gd_align16(GD_LANE_WORDS * 4);
  b += gd_align16(GD_SW * 4);
  b += gd_align16(GD_SW * 2);
  b += gd_align16(16 * 4);
  b += gd_align16(256 * 8);
  b += gd_align16(GD_OBS * GD_OBS);
  b += gd_align16(64);
  b += gd_align16(14 * GD_SW * 4);
  b += 2 * gd_align16(GD_SW * 4);
  b += gd_align16(256 * 4);
  b += 2 * gd_align16(8 * GD_SW * 4) + gd_align16(8 * GD_SW);
  b += gd_align16((size_t)W * sizeof(GdWall));
  b += gd_align16((size_t)(maxThings > 0 ? maxThings : 1) * sizeof(GdActor));
  return b;
}

__device__ inline void gd_carve(uint8_t *base, int W, int maxThings, GdShared &s) {
  size_t o = 0;
  s.frame = base + o; o += gd_align16((size_t)GD_SCREEN_H * GD_SW);
  s.colormap = base + o; o += gd_align16(32 * 256);
  s.playpal = base + o; o += gd_align16(768);
  s.yslope = (unsigned *)(base + o); o += gd_align16(GD_VH * 4);
  s.lane = (int32_t *)(base + o); o += gd_align16(GD_LANE_WORDS * 4);
  s.wallDistance = (float *)(base + o); o += gd_align16(GD_SW * 4);
  s.blockingWall = (short *)(base + o); o += gd_align16(GD_SW * 2);
  s.ownerMask = (unsigned *)(base + o); o += gd_align16(16 * 4);
  s.pal64 = (unsigned long long *)(base + o); o += gd_align16(256 * 8);
  s.obs = base + o; o += gd_align16(GD_OBS * GD_OBS);
  s.misc = (int *)(base + o); o += gd_align16(64);
  s.masks = (unsigned *)(base + o); o += gd_align16(14 * GD_SW * 4);
  s.maskedDist = (float *)(base + o); o += gd_align16(GD_SW * 4);
  s.maskedInfo = (unsigned *)(base + o); o += gd_align16(GD_SW * 4);
  s.pal32 = (unsigned *)(base + o); o += gd_align16(256 * 4);
  s.hitD = (float *)(base + o); o += gd_align16(8 * GD_SW * 4);
  s.hitA = (float *)(base + o); o += gd_align16(8 * GD_SW * 4);
  s.hitF = base + o; o += gd_align16(8 * GD_SW);
  s.walls = (GdWall *)(base + o); o += gd_align16((size_t)W * sizeof(GdWall));
  s.actors = (GdActor *)(base + o);
}

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

/* Project wall w of the map for this lane (engine.py:10747-10869, 11207-11302,
 * 11359-11427).  The ray-owned span is completed by gd_wall_span below. */
__device__ __noinline__ void gd_project_wall(const GdScene &sc, const GdView &v, int w, GdWall &out) {
  const float *wl = &sc.walls[w * 4];
  i64 fx[2] = {gd_rint(wl[0] * 65536.0f), gd_rint(wl[2] * 65536.0f)};
  i64 fy[2] = {gd_rint(wl[1] * 65536.0f), gd_rint(wl[3] * 65536.0f)};
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
  out.oneSided = sc.wsec[w * 2 + 1] < 0;
  float sx = wl[0], sy = wl[1];
  float segx = wl[2] - sx, segy = wl[3] - sy;
  float vfsx = v.x - sx, vfsy = v.y - sy;
  out.frontF = (segx * vfsy - segy * vfsx) < 0;
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

__device__ __noinline__ GdHit gd_hit_slow(const GdScene &sc, const GdView &v, const GdWall *walls, int w, int x,
                                          float rx, float ry) {
  return gd_hit(sc, v, walls, w, x, rx, ry);
}

__device__ __forceinline__ float gd_tol(float d) { return fmaxf(fabsf(d) / 128.0f, 4.0f); }

/* Endpoint owner of wall w at column x (engine.py:11589-11730). */
__device__ __noinline__ void gd_endpoint_owner(const GdScene &sc, const GdView &v, const GdWall *walls, int w, int x, float rx,
                                  float ry, const GdHit &hw, int &ownerIdx, float &ownerDist) {
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
    int sIdx = nd[0] >= 0 ? nd[0] : w, eIdx = nd[1] >= 0 ? nd[1] : w;
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
      int nb = sc.nbIdx[k], fl = sc.nbFlags[k];
      GdHit hn = gd_hit(sc, v, walls, nb, x, rx, ry);
      bool rayNb = usesStart ? (fl & 1) : ((fl >> 1) & 1);
      bool sel = rayNb || (subpixel && (fabsf(hn.d - d) <= tol));
      float cand = (hn.proj && hn.left && sel) ? hn.d : GD_INF;
      if (cand < best) { best = cand; bestSlot = k - n0; }
    }
    od = best;
    oi = (n1 > n0) ? sc.nbIdx[n0 + bestSlot] : w;
    ownerValid = isfinite(best);
  }
  bool has = !hw.proj && ownerValid;
  ownerIdx = has ? oi : w;
  ownerDist = has ? od : d;
}

/* PrepWall for one (column, wall) (engine.py:10672-10739). */
__device__ __noinline__ void gd_prep_wall(const GdScene &sc, const GdWall &wv, int w, int x, i64 &hoff, i64 &vstep) {
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
__device__ __noinline__ int gd_project_rows(const GdView &v, const GdWall &wv, float worldZ, int x) {
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

/* Column-independent part of gd_project_rows for one (wall, height). */
__device__ __noinline__ void gd_rowproj_setup(const GdView &v, const GdWall &wv, float worldZ, GdRowProj &o) {
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
__device__ __forceinline__ int gd_secidx(const GdScene &sc, int s) { return s < 0 ? s + sc.S : s; }
__device__ __forceinline__ float gd_sec_floor(const GdScene &sc, int s) { return sc.secF[gd_secidx(sc, s) * 2]; }
__device__ __forceinline__ float gd_sec_ceil(const GdScene &sc, int s) { return sc.secF[gd_secidx(sc, s) * 2 + 1]; }
__device__ __forceinline__ int4 gd_sec_info(const GdScene &sc, int s) {
  return *reinterpret_cast<const int4 *>(&sc.secI[gd_secidx(sc, s) * 4]);
}

__device__ __forceinline__ bool gd_same_pair(const GdScene &sc, int a, int b) {
  int a0 = sc.wsec[a * 2], a1 = sc.wsec[a * 2 + 1], b0 = sc.wsec[b * 2], b1 = sc.wsec[b * 2 + 1];
  return (a0 == b0 && a1 == b1) || (a0 == b1 && a1 == b0);
}
__device__ __forceinline__ bool gd_shares_endpoint(const GdScene &sc, int a, int b) {
  int a0 = sc.wvtx[a * 2], a1 = sc.wvtx[a * 2 + 1], b0 = sc.wvtx[b * 2], b1 = sc.wvtx[b * 2 + 1];
  return a0 == b0 || a0 == b1 || a1 == b0 || a1 == b1;
}
__device__ __noinline__ bool gd_opposing_pair(const GdScene &sc, int a, int b) {
  if (!gd_same_pair(sc, a, b)) return false;
  if (sc.wsec[a * 2 + 1] < 0 || sc.wsec[b * 2 + 1] < 0) return false;
  if (gd_shares_endpoint(sc, a, b)) return false;
  const float *A = &sc.walls[a * 4], *B = &sc.walls[b * 4];
  float adx = A[2] - A[0], ady = A[3] - A[1], bdx = B[2] - B[0], bdy = B[3] - B[1];
  float dot = adx * bdx + ady * bdy;
  float cross = adx * bdy - ady * bdx;
  return dot < 0 && fabsf(cross) < 1e-6f;
}
__device__ __forceinline__ bool gd_two_distinct(const GdScene &sc, int w) {
  return sc.wsec[w * 2 + 1] >= 0 && sc.wsec[w * 2] != sc.wsec[w * 2 + 1];
}
__device__ bool gd_bridge_pair_of(const GdScene &sc, int a, int b, int &p0, int &p1) {
  int a0 = sc.wsec[a * 2], a1 = sc.wsec[a * 2 + 1], b0 = sc.wsec[b * 2], b1 = sc.wsec[b * 2 + 1];
  int shared = 0, sv = -2;
  if (a0 == b0 || a0 == b1) { shared++; sv = a0; }
  if (a1 == b0 || a1 == b1) { shared++; sv = a1; }
  if (shared != 1) return false;
  p0 = (a0 == sv) ? a1 : a0;
  p1 = (b0 == sv) ? b1 : b0;
  return true;
}
__device__ __forceinline__ bool gd_set_equals(const GdScene &sc, int w, int p0, int p1) {
  int s0 = sc.wsec[w * 2], s1 = sc.wsec[w * 2 + 1];
  if (p0 == p1) return s0 == p0 && s1 == p0;
  return (s0 == p0 && s1 == p1) || (s0 == p1 && s1 == p0);
}
__device__ bool gd_unique_at_vertex(const GdScene &sc, int v, int skipA, int skipB, int p0, int p1, int &index) {
  int count = 0, found = 0;
#pragma unroll 1
  for (int k = sc.vtxOff[v]; k < sc.vtxOff[v + 1]; ++k) {
    int c = sc.vtxWalls[k];
    if (c == skipA || c == skipB) continue;
    if (gd_set_equals(sc, c, p0, p1)) { count++; found = c; }
  }
  index = (count == 1) ? found : 0;
  return count == 1;
}
__device__ __noinline__ bool gd_portal_bridge(const GdScene &sc, int slot, int path, int owner, int &index) {
  index = 0;
  if (!gd_two_distinct(sc, path) || owner == path) return false;
  int v = sc.wvtx[path * 2 + slot];
  if (sc.wvtx[owner * 2] != v && sc.wvtx[owner * 2 + 1] != v) return false;
  if (!gd_two_distinct(sc, owner)) return false;
  int p0, p1;
  if (!gd_bridge_pair_of(sc, path, owner, p0, p1)) return false;
  return gd_unique_at_vertex(sc, v, path, owner, p0, p1, index);
}
__device__ __noinline__ bool gd_sector_bridge(const GdScene &sc, int slot, int pending, int path, int &index) {
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

__device__ void gd_wall_spans(const GdScene &sc, const GdView &v, const GdShared &sh) {
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
__device__ void gd_blocking_raycast(const GdScene &sc, const GdView &v, const GdShared &sh, const short *list, int listed,
                                    float rx, float ry, float &wallDistance, int &blockingWall) {
  float best = GD_INF;
  int bestWall = sc.blocking[0];
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

/* ---- visplane rows (engine.py:10879-10954, 10588-10616, 13372-13405) ---- */
struct GdPlaneSpan {
  i64 basex, basey, pviewx, pviewy, phf, gv, shadeBase;
  const uint8_t *tex;
  int wbits, hbits, texW;
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

__device__ __noinline__ void gd_plane_entry_setup(const GdScene &sc, const GdView &v, int sector, bool isFloor,
                                                  GdPlaneEntry &e) {
  float ph = isFloor ? (v.viewZ - gd_sec_floor(sc, sector)) : (gd_sec_ceil(sc, sector) - v.viewZ);
  int4 si = gd_sec_info(sc, sector);
  int tex = isFloor ? si.y : si.z;
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
}

__device__ __forceinline__ void gd_plane_setup(const GdScene &sc, const GdPlaneEntry *table, int sector, bool isFloor,
                                               int x, GdPlaneSpan &p) {
  const GdPlaneEntry &e = table[gd_secidx(sc, sector) * 2 + (isFloor ? 1 : 0)];
  i64 col = (i64)x - 159;
  p.wbits = e.wbits; p.hbits = e.hbits; p.texW = sc.texW;
  p.tex = e.tex;
  p.basex = e.bx0 + col * e.xstep;
  p.basey = e.by0 + col * e.ystep;
  p.pviewx = e.pviewx;
  p.pviewy = e.pviewy;
  p.phf = e.phf;
  p.gv = e.gv;
  p.shadeBase = e.shadeBase;
}

__device__ __forceinline__ uint8_t gd_plane_pixel(const GdPlaneSpan &p, const GdView &v, const unsigned *yslope,
                                                  const uint8_t *colormap, int y) {
  i64 distance = gd_wmul(p.phf, (i64)yslope[y]) >> 16;
  i64 xfrac = ((gd_wmul(distance, p.basex) >> 16) + p.pviewx) & GD_U32MASK;
  i64 yfrac = ((gd_wmul(distance, p.basey) >> 16) + p.pviewy) & GD_U32MASK;
  int u = (int)(xfrac >> (32 - p.wbits)), tv = (int)(yfrac >> (32 - p.hbits));
  uint8_t texel = p.tex[tv * p.texW + u];
  i64 rowDist = v.center - (i64)y * GD_FU;
  if (rowDist < 0) rowDist = -rowDist;
  i64 vis = gd_min(gd_wmul(p.gv, rowDist) >> 16, 24 * GD_FU);
  int shade = (int)gd_clamp((p.shadeBase - vis) >> 16, 0, 31);
  return colormap[shade * 256 + texel];
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

#ifdef GD_PROFILE_PHASES
__device__ unsigned long long *gdProfile;   /* decide-phase cycle counters */
#define GD_TD(m) do { if ((x & 31) == 0) { long long t = clock64(); atomicAdd(gdProfile + 32 + (m), (unsigned long long)(t - gdD0)); gdD0 = t; } } while (0)
#else
#define GD_TD(m) do {} while (0)
#endif

__device__ void gd_column_decide(const GdScene &sc, const GdView &v, const GdWall *walls, const unsigned *ownerMask,
                                 const GdRowProj *rowproj, float *hitD, float *hitA, uint8_t *hitF, int x, float rx,
                                 float ry, const GdColState &c, GdIter &it) {
  const int curSector = c.cur;
  const int current = curSector < 0 ? 0 : curSector;
  const float prev = c.prev;
  const int i0 = sc.secOff[current], i1 = sc.secOff[current + 1];
#ifdef GD_PROFILE_PHASES
  long long gdD0 = clock64();
#endif
  /* every rule below looks at the walls of the current sector: test each once
   * and keep the results in this column's slice of shared memory */
  constexpr int kCache = 8;
  const int nCache = min(i1 - i0, kCache);
#pragma unroll 1
  for (int k = 0; k < nCache; ++k) {
    GdHit h = gd_hit(sc, v, walls, sc.secWalls[i0 + k], x, rx, ry);
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
#define HITK(k) (((k) - i0) < nCache ? loadHit((k) - i0) : gd_hit_slow(sc, v, walls, sc.secWalls[k], x, rx, ry))
  float distance = GD_INF;
  int wallIndex = 0;
  if (curSector >= 0) {
#pragma unroll 1
    for (int k = i0; k < i1; ++k) {
      int w = sc.secWalls[k];
      GdHit h = HITK(k);
      if (h.d > prev && h.d < distance) { distance = h.d; wallIndex = w; }
    }
    float sd = GD_INF;
    int sw = 0;
#pragma unroll 1
    for (int k = i0; k < i1; ++k) {
      int w = sc.secWalls[k];
      if (!walls[w].oneSided) continue;
      GdHit h = HITK(k);
      if (!(h.d > prev) || !isfinite(h.d)) continue;
      if (fabsf(h.d - distance) <= 1e-3f && h.d < sd) { sd = h.d; sw = w; }
    }
    if (isfinite(sd)) { distance = sd; wallIndex = sw; }
  }
  GD_TD(1);
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
      int w = sc.secWalls[k];
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
        int b = idx[k];
        bool inc = sc.wsec[b * 2] == current || sc.wsec[b * 2 + 1] == current;
        if (!inc || !walls[b].oneSided) continue;
        GdHit h = HIT(b);
        if (h.proj && h.left && (h.d > prev + 1e-3f) && h.d < sbd) { sbd = h.d; sbi = b; }
      }
      if (sbd < psd) { psd = sbd; psi = sbi; }
    }
  }
  GD_TD(2);
  bool hasProjectedSolidOwner = isfinite(psd);
  if (hasProjectedSolidOwner) { distance = psd; wallIndex = psi; }
  GdHit hW = (wallIndex == psPathIndex) ? hSel : HIT(wallIndex);
  int seo = wallIndex;
  float sed = hW.d;
  if (!hW.proj) gd_endpoint_owner(sc, v, walls, wallIndex, x, rx, ry, hW, seo, sed);
  bool eoPathIsGeo = hW.geo;
  bool replaceEo = (seo != wallIndex) && (sed > prev + 1e-3f);
  if (replaceEo) { distance = sed; wallIndex = seo; hW = HIT(wallIndex); }
  GD_TD(3);
  int nopIndex = wallIndex;
  float nopDist = distance;
  bool nopIsGeo = replaceEo ? eoPathIsGeo : hW.geo;
  bool nopFromFront = curSector == sc.wsec[nopIndex * 2];
  int nopOther = nopFromFront ? sc.wsec[nopIndex * 2 + 1] : sc.wsec[nopIndex * 2];
  bool selOwnerIsProjected = hW.proj;
  bool selOwnerExclRight = walls[wallIndex].sr == x;
  i64 selOwnerSpan = walls[wallIndex].sr - walls[wallIndex].sl;
  bool selOwnerShort = sc.wlen[wallIndex] <= 32.0f;
  float npd = GD_INF;
  int npi = 0;
  if (!selOwnerIsProjected) {
#pragma unroll 1
    for (int k = i0; k < i1; ++k) {
      int w = sc.secWalls[k];
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
  bool peFromCur = curSector == sc.wsec[pew * 2];
  int peOther = peFromCur ? sc.wsec[pew * 2 + 1] : sc.wsec[pew * 2];
  bool usePsb = false;
  if (c.pendEpBoundary && !selOwnerIsProjected && selOwnerExclRight && nopIsGeo) {
    bool peIncident = peFromCur || curSector == sc.wsec[pew * 2 + 1];
    const float *peWall = &sc.walls[pew * 4];
    int peSlot = (c.pendEpEpX == peWall[2] && c.pendEpEpY == peWall[3]) ? 1 : 0;
    int psbIndex;
    bool psbExists = gd_sector_bridge(sc, peSlot, pew, nopIndex, psbIndex);
    if (psbExists && peIncident && peOther >= 0 && nopOther >= 0 && (walls[pew].sr - walls[pew].sl <= 1)) {
      int b0 = sc.wsec[psbIndex * 2], b1 = sc.wsec[psbIndex * 2 + 1];
      bool matches = (b0 == peOther && b1 == nopOther) || (b1 == peOther && b0 == nopOther);
      GdHit hb = HIT(psbIndex);
      GdHit hp = HIT(pew);
      bool psb = matches && hb.proj && hb.left && (hb.d > prev - gd_tol(hp.d)) && (hb.d < nopDist);
      if (psb && hb.d < npd) { usePsb = true; npd = hb.d; npi = psbIndex; }
    }
  }
  GD_TD(4);
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
  int front = sc.wsec[wallIndex * 2], back = sc.wsec[wallIndex * 2 + 1];
  bool fromFront = curSector == front;
  int otherSector = fromFront ? back : front;
  int renderCurrent = usePsb ? peOther : (completesOpposing ? otherSector : current);
  bool renderFromFront = renderCurrent == front;
  int renderOther = renderFromFront ? back : front;
  int side = renderFromFront ? 0 : 1;
  const GdWall &wv = walls[wallIndex];
  i64 vis = wv.visL[side] + ((i64)x - wv.visSl[side]) * wv.visStep[side];
  bool psFromFront = curSector == sc.wsec[psPathIndex * 2];
  int psOther = psFromFront ? sc.wsec[psPathIndex * 2 + 1] : sc.wsec[psPathIndex * 2];
  bool pskpp = hasProjectedSolidOwner && hSel.geo && psOther >= 0;
  int safeOther = renderOther < 0 ? 0 : renderOther;
  float viewFloor = gd_sec_floor(sc, renderCurrent), viewCeil = gd_sec_ceil(sc, renderCurrent);
  float otherFloor = gd_sec_floor(sc, safeOther), otherCeil = gd_sec_ceil(sc, safeOther);
  bool oneSided = otherSector < 0;
  const int32_t *stex = &sc.sideTex[(wallIndex * 2 + side) * 3];
  GD_TD(5);
  /* Row bounds: per (wall, sector height) tables built once per lane cover the
   * usual case of heights taken from the wall's own two sectors. */
  const GdRowProj *rp = rowproj + wallIndex * 4;
  int slotCur = (renderCurrent == front) ? 0 : ((renderCurrent == back && back >= 0) ? 2 : -1);
  int oneTop = 0, oneBottom = 0;
  /* the row bounds feed tiers, marks, clips and events, all of which need a
   * raster-valid crossing */
  if (!rasterValid) {
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
    if (slotOther >= 0) {
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

  GD_TD(6);
  /* traversal decisions (engine.py:13070-13241) */
  bool endpointOnly = valid && !oneSided && !geometric;
  float cnd = GD_INF, ond = GD_INF, csd = GD_INF, osd = GD_INF, gpd = GD_INF;
  int cni = 0, oni = 0, gpi = 0;
  const float prior = prev;
  if (endpointOnly) {
#pragma unroll 1
    for (int k = i0; k < i1; ++k) {
      int w = sc.secWalls[k];
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
      int w = sc.secWalls[k];
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
  bool gpFromFront = curSector == sc.wsec[gpi * 2];
  int gpOther = gpFromFront ? sc.wsec[gpi * 2 + 1] : sc.wsec[gpi * 2];
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
  GD_TD(7);
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

__device__ __noinline__ void gd_draw_tier(const GdScene &sc, const GdView &v, const GdShared &sh, int x, int ya, int yb, int ea,
                             int eb, int texId, float originZ, const GdTierCtx &t, i64 vis, i64 firstVis,
                             bool tailValid, int tailBottom, int oa, int ob, bool oTailValid, int oTailBottom,
                             unsigned *filled) {
  if (texId < 0 || ya >= yb) return;
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
  const uint8_t *cmN = sh.colormap + shadeN * 256, *cmT = sh.colormap + shadeT * 256;
  /* rows lit with the group's first-column light */
  const int tailA = tailValid ? tailBottom : GD_VH, oTailA = oTailValid ? max(oa, oTailBottom) : 0,
            oTailB = oTailValid ? ob : 0;
  const int shift = 32 - hbits;
  uint8_t *dst = sh.frame + x;
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
      uint8_t t0 = col[f0 >> shift], t1 = col[f1 >> shift];
      uint8_t p0 = ((tailM >> b0) & 1u ? cmT : cmN)[t0], p1 = ((tailM >> b1) & 1u ? cmT : cmN)[t1];
      dst[(y0 + b0) * GD_SW] = p0;
      dst[(y0 + b1) * GD_SW] = p1;
    }
  }
}

__device__ __noinline__ void gd_mark_plane(const GdScene &sc, const GdView &v, const GdShared &sh, int x, int ya, int yb,
                              int sector, bool isFloor, unsigned *owned, const unsigned *filled) {
  if (ya >= yb) return;
  const int k0 = ya >> 5, k1 = (yb - 1) >> 5;
  unsigned any = 0;
#pragma unroll 1
  for (int k = k0; k <= k1; ++k) any |= gd_range_word(k, ya, yb) & ~owned[k * GD_SW];
  if (!any) return;
  GdPlaneSpan p;
  gd_plane_setup(sc, sh.planeTab, sector, isFloor, x, p);
  uint8_t *dst = sh.frame + x;
#pragma unroll 1
  for (int k = k0; k <= k1; ++k) {
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
      uint8_t p0 = gd_plane_pixel(p, v, sh.yslope, sh.colormap, y0 + b0);
      uint8_t p1 = gd_plane_pixel(p, v, sh.yslope, sh.colormap, y0 + b1);
      dst[(y0 + b0) * GD_SW] = p0;
      dst[(y0 + b1) * GD_SW] = p1;
    }
  }
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

__device__ __noinline__ void gd_masked_pass(const GdScene &sc, const GdView &v, const GdShared &sh) {
  const int x = threadIdx.x;
  float rx, ry;
  gd_ray(v, x, rx, ry);
  float best = GD_INF;
  int w = -1, side = 0, texId = -1;
  bool leftEdge = false;
#pragma unroll 1
  for (int i = 0; i < sc.M; ++i) {
    const int k = sc.maskedWalls[i];
    const int sd = sh.walls[k].frontF ? 0 : 1;
    const int t = sc.sideTex[(k * 2 + sd) * 3];
    if (t < 0) continue;
    GdHit h = gd_hit_slow(sc, v, sh.walls, k, x, rx, ry);
    if (h.proj && h.d < best) { best = h.d; w = k; side = sd; texId = t; leftEdge = h.left; }
  }
  if (!isfinite(best)) return;
  const GdWall &wv = sh.walls[w];
  const int front = sc.wsec[w * 2], back = sc.wsec[w * 2 + 1] < 0 ? 0 : sc.wsec[w * 2 + 1];
  const int lightSector = side == 0 ? front : back;
  const float worldTop = fminf(gd_sec_ceil(sc, front), gd_sec_ceil(sc, back));
  const int4 ti = *reinterpret_cast<const int4 *>(&sc.texInfo[texId * 4]);
  const int tw = ti.x, th = ti.y, hbits = ti.w;
  const i64 owallTop = gd_project_rows(v, wv, worldTop, x);
  const i64 owallBottom = gd_project_rows(v, wv, worldTop - (float)th, x);
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
  if (!(hasSaved || leftEdge)) return;
  const float *wl = &sc.walls[w * 4];
  const bool horizontal = fabsf(wl[3] - wl[1]) < 1e-6f, vertical = fabsf(wl[2] - wl[0]) < 1e-6f;
  const i64 light = gd_sec_info(sc, lightSector).x + v.flashLight * 16 + (vertical ? 16 : (horizontal ? -16 : 0));
  const i64 vis = wv.visL[side] + ((i64)x - wv.visSl[side]) * wv.visStep[side];
  const uint8_t *cm = sh.colormap + gd_wall_shade(light, vis) * 256;
  const uint8_t *col = sc.texAtlasCol + ((size_t)texId * sc.texW + u) * sc.texH;
  const unsigned base = (unsigned)(gd_shl(texMid, 16 - hbits) + (gd_wmul(vstep, GD_FU - v.center) >> 16));
  const unsigned step = (unsigned)vstep;
#pragma unroll 1
  for (int y = (int)gd_max(clippedTop, 0); y < (int)gd_min(clippedBottom, GD_VH); ++y)
    sh.frame[y * GD_SW + x] = cm[col[(base + (unsigned)y * step) >> (32 - hbits)]];
}

#define GD_FALLBACK_MAX (8 * GD_SW)

__device__ void gd_walk(const GdScene &sc, const GdView &v, const GdShared &sh, GdEvent *events, int *eventCount,
                        const GdRowProj *rowproj, int *status, int startSector) {
  const int x = threadIdx.x;
  const int lane = x & 31;
  const unsigned quadBase = lane & ~3u;
  float rx, ry;
  gd_ray(v, x, rx, ry);
  unsigned *filled = sh.masks + x, *owned = sh.masks + 7 * GD_SW + x;
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
#ifdef GD_PROFILE_PHASES
  long long gdW0 = clock64();
#endif
  int nEvents = 0;
  bool overflow = false;

  for (int iter = 0; iter < sc.S; ++iter) {
    if (__all_sync(0xffffffffu, settled)) break;
#ifdef GD_PROFILE_PHASES
#define GD_TB(m) do { if ((x & 31) == 0) { long long t = clock64(); atomicAdd((unsigned long long *)(status + 8) + 16 + (m), (unsigned long long)(t - gdW0)); gdW0 = t; } } while (0)
#else
#define GD_TB(m) do {} while (0)
#endif
    GD_TB(0);
#ifdef GD_PROFILE_PHASES
    if ((x & 31) == 0) atomicAdd((unsigned long long *)(status + 8) + 24, 1ull);
    if (!settled) atomicAdd((unsigned long long *)(status + 8) + 25, 1ull);
    if (!settled && c.cur >= 0) atomicAdd((unsigned long long *)(status + 8) + 26, 1ull);
#endif
    GdIter it;
    if (!settled) {
      gd_column_decide(sc, v, sh.walls, sh.ownerMask, rowproj, sh.hitD, sh.hitA, sh.hitF, x, rx, ry, c, it);
    } else {
      it.wall = -1 - x; it.side = 0; it.tier[0] = it.tier[1] = it.tier[2] = false;
      it.ctop = it.clowtop = 0; it.cbot = it.cupbot = 0; it.vis = 0;
      it.rasterValid = false; it.valid = false; it.pskpp = false;
    }
    GD_TB(1);
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
    GD_TB(2);
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
      GD_TB(3);
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
    GD_TB(4);
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
      const GdWall &pw = sh.walls[pIdx];
      int pSafeOther = it.psOther < 0 ? 0 : it.psOther;
      float pOtherFloor = gd_sec_floor(sc, pSafeOther), pOtherCeil = gd_sec_ceil(sc, pSafeOther);
      int pSide = it.psFromFront ? 0 : 1;
      const int32_t *ptex = &sc.sideTex[(pIdx * 2 + pSide) * 3];
      int pTop = gd_project_rows(v, pw, it.viewCeil, x), pBottom = gd_project_rows(v, pw, it.viewFloor, x);
      int pLowerTop = gd_project_rows(v, pw, pOtherFloor, x), pUpperBottom = gd_project_rows(v, pw, pOtherCeil, x);
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
    GD_TB(5);
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
    GD_TB(6);
  }
  eventCount[x] = nEvents < GD_MAX_EVENTS ? nEvents : GD_MAX_EVENTS;
  if (overflow) atomicOr(status, GD_STATUS_EVENT_OVERFLOW);

}

/* ---- point in sector (engine.py:9598-9617) ------------------------------ */
/* Crossing parity of a +x ray over the sector's edges.  The bounding box only
 * skips sectors whose parity is provably even. */
__device__ __forceinline__ bool gd_point_in_sector(const GdScene &sc, int s, float px, float py) {
  const float4 bb = *reinterpret_cast<const float4 *>(&sc.secBBox[s * 4]);
  if (py >= bb.w || py < bb.z) return false;           /* no edge straddles the ray's row */
  if (px > bb.y + 1.0f) return false;                  /* every crossing lies left of the point */
  if (px < bb.x - 1.0f && sc.secI[s * 4 + 3]) return false;  /* closed loops cross an even number of times */
  int crossings = 0;
#pragma unroll 1
  for (int k = sc.edgeOff[s]; k < sc.edgeOff[s + 1]; ++k) {
    const float4 e = *reinterpret_cast<const float4 *>(&sc.walls[sc.edgeWalls[k] * 4]);
    bool crosses = (e.y > py) != (e.w > py);
    float dy = e.w - e.y;
    float safe = fabsf(dy) < 1e-6f ? 1.0f : dy;
    float cx = e.x + (py - e.y) * (e.z - e.x) / safe;
    crossings += (crosses && (px < cx)) ? 1 : 0;
  }
  return crossings & 1;
}

/* Flat-fallback resolution of a pixel (engine.py:10961-11026): true when the
 * column ray meets no sector's plane inside that sector's polygon. */
__device__ __noinline__ bool gd_pixel_unresolved(const GdScene &sc, const GdView &v, int x, int y, float rc, float rs,
                                                 int hint) {
  i64 ti = gd_clamp((GD_ANG90 - v.pitchBam) >> 19, 0, 4095);
  i64 offFixed = ((i64)sc.fineTan[ti] * 12582912LL) >> 16;
  float center = 103.5f + (float)offFixed / 65536.0f;
  float cc = sc.rayCosCorr[x];
  float delta = (float)y - center;
  bool floorPixel = delta > 0;
  float den = fmaxf(fabsf(delta), 0.5f);
  /* An existence test, so the order is free: `hint` (the sector whose plane
   * was marked on this pixel) is nearly always the one that answers it; the
   * others are visited by plane height, one plane point per distinct height. */
  {
    float ph = floorPixel ? (v.viewZ - sc.secF[hint * 2]) : (sc.secF[hint * 2 + 1] - v.viewZ);
    float cd = ph * 192.0f / den / cc;
    if (ph > 0 && isfinite(cd) && cd > 0 && gd_point_in_sector(sc, hint, v.x + rc * cd, v.y + rs * cd)) return false;
  }
  const int f = floorPixel ? 1 : 0;
  const float *gh = sc.groupH[f];
  const int32_t *goff = sc.groupOff[f], *gsec = sc.groupSec[f];
#pragma unroll 1
  for (int g = 0; g < sc.groups[f]; ++g) {
    float ph = floorPixel ? (v.viewZ - gh[g]) : (gh[g] - v.viewZ);
    float perp = ph * 192.0f / den;
    float cd = perp / cc;
    if (!(ph > 0) || !isfinite(cd) || !(cd > 0)) continue;
    float px = v.x + rc * cd, py = v.y + rs * cd;
#pragma unroll 1
    for (int k = goff[g]; k < goff[g + 1]; ++k)
      if (gd_point_in_sector(sc, gsec[k], px, py)) return false;
  }
  return true;
}

__device__ float gd_plane_depth(const GdScene &sc, const GdView &v, int sector, bool isFloor, int y) {
  i64 ti = gd_clamp((GD_ANG90 - v.pitchBam) >> 19, 0, 4095);
  i64 offFixed = ((i64)sc.fineTan[ti] * 12582912LL) >> 16;
  float flatCenter = (103.0f + (float)offFixed / 65536.0f) + 0.5f;
  float ph = isFloor ? (v.viewZ - gd_sec_floor(sc, sector)) : (gd_sec_ceil(sc, sector) - v.viewZ);
  float den = fmaxf(fabsf((float)y - flatCenter), 0.5f);
  return ph * 192.0f / den;
}

__device__ __forceinline__ float gd_wrap_angle(float a) {
  const float pi = 3.14159265358979323846f, twoPi = 6.28318530717958647692f;
  float t = a + pi;
  float r = fmodf(t, twoPi);
  if (r != 0 && (r < 0)) r += twoPi;
  return r - pi;
}

/* ---- per-pixel flat fallback (engine.py:10956-11171) ------------------------
 * Only pixels that no seg and no visplane claimed show this layer, so it is
 * evaluated lazily for exactly those pixels.  The reference resolves every
 * pixel, repairs unresolved ones from the next resolved row below and then
 * from the nearest anchors left and right; the scans below visit only the
 * pixels those repairs would read for the one pixel asked for. */
struct GdFlatProbe { bool unresolved, isFloor; int sector; };

/* the part of a probe that depends on the column only */
struct GdFlatRay { float rc, rs, cc, center; };

/* Per-lane bounds that let a probe prove "no sector" without visiting any:
 * the smallest positive plane height of either orientation (the nearest plane
 * point of every sector lies at least that far along the ray) and the box
 * outside which gd_point_in_sector rejects every sector. */
struct GdFlatBounds { float phFloor, phCeil, xHi, xLo, yHi, yLo; int allClosed; };

__device__ __forceinline__ GdFlatBounds gd_flat_bounds_load(const int *misc) {
  GdFlatBounds b;
  b.phFloor = __int_as_float(misc[4]); b.phCeil = __int_as_float(misc[5]);
  b.xHi = __int_as_float(misc[6]); b.xLo = __int_as_float(misc[7]);
  b.yHi = __int_as_float(misc[8]); b.yLo = __int_as_float(misc[9]);
  b.allClosed = misc[10];
  return b;
}

/* warp 0 fills misc[4..10] */
__device__ void gd_flat_bounds_setup(const GdScene &sc, const GdView &v, int *misc) {
  const int lane = threadIdx.x & 31;
  float phF = GD_INF, phC = GD_INF, xHi = -GD_INF, xLo = GD_INF, yHi = -GD_INF, yLo = GD_INF;
  int closed = 1;
  for (int s = lane; s < sc.S; s += 32) {
    float f = v.viewZ - sc.secF[s * 2], c = sc.secF[s * 2 + 1] - v.viewZ;
    if (f > 0) phF = fminf(phF, f);
    if (c > 0) phC = fminf(phC, c);
    const float4 bb = *reinterpret_cast<const float4 *>(&sc.secBBox[s * 4]);
    xHi = fmaxf(xHi, bb.y + 1.0f);
    xLo = fminf(xLo, bb.x - 1.0f);
    yHi = fmaxf(yHi, bb.w);
    yLo = fminf(yLo, bb.z);
    closed &= sc.secI[s * 4 + 3] != 0;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    phF = fminf(phF, __shfl_xor_sync(0xffffffffu, phF, o));
    phC = fminf(phC, __shfl_xor_sync(0xffffffffu, phC, o));
    xHi = fmaxf(xHi, __shfl_xor_sync(0xffffffffu, xHi, o));
    xLo = fminf(xLo, __shfl_xor_sync(0xffffffffu, xLo, o));
    yHi = fmaxf(yHi, __shfl_xor_sync(0xffffffffu, yHi, o));
    yLo = fminf(yLo, __shfl_xor_sync(0xffffffffu, yLo, o));
    closed &= __shfl_xor_sync(0xffffffffu, closed, o);
  }
  if (lane == 0) {
    misc[4] = __float_as_int(phF); misc[5] = __float_as_int(phC);
    misc[6] = __float_as_int(xHi); misc[7] = __float_as_int(xLo);
    misc[8] = __float_as_int(yHi); misc[9] = __float_as_int(yLo);
    misc[10] = closed;
  }
}

__device__ __noinline__ GdFlatRay gd_flat_ray(const GdScene &sc, const GdView &v, int x) {
  i64 ti = gd_clamp((GD_ANG90 - v.pitchBam) >> 19, 0, 4095);
  i64 offFixed = ((i64)sc.fineTan[ti] * 12582912LL) >> 16;
  GdFlatRay r;
  r.center = 103.5f + (float)offFixed / 65536.0f;
  float rayAngle = v.angle + sc.rayOffsets[x];
  r.rc = cosf(rayAngle);
  r.rs = sinf(rayAngle);
  r.cc = sc.rayCosCorr[x];
  return r;
}

__device__ __noinline__ GdFlatProbe gd_flat_probe(const GdScene &sc, const GdView &v, const GdFlatRay &r,
                                                  const GdFlatBounds &b, int y, int currentSector) {
  float delta = (float)y - r.center;
  GdFlatProbe out;
  out.isFloor = delta > 0;
  float den = fmaxf(fabsf(delta), 0.5f);
  out.sector = currentSector;
  out.unresolved = true;
  {
    /* Every sector's plane point lies at cd >= cd0 along the ray, and each
     * coordinate moves monotonically with cd (the roundings are monotone too):
     * once the nearest candidate is past the box on the side the ray is
     * heading to, every sector rejects every candidate. */
    float ph0 = out.isFloor ? b.phFloor : b.phCeil;
    float cd0 = ph0 * 192.0f / den / r.cc;
    if (!isfinite(cd0)) return out;
    if (cd0 > 0) {
      float px0 = v.x + r.rc * cd0, py0 = v.y + r.rs * cd0;
      if (r.rc > 0 && px0 > b.xHi) return out;
      if (r.rc < 0 && b.allClosed && px0 < b.xLo) return out;
      if (r.rs > 0 && py0 >= b.yHi) return out;
      if (r.rs < 0 && py0 < b.yLo) return out;
    }
  }
  /* Sectors are visited by plane height, nearest plane first, so the distance
   * along the ray never decreases from group to group: the first group with a
   * sector that contains its plane point holds the answer, except that a later
   * group whose distance rounds to the same value may still own it with a lower
   * sector index (the reference keeps the first index among equal distances). */
  float best = GD_INF;
  const int f = out.isFloor ? 1 : 0;
  const float *gh = sc.groupH[f];
  const int32_t *goff = sc.groupOff[f], *gsec = sc.groupSec[f];
#pragma unroll 1
  for (int g = 0; g < sc.groups[f]; ++g) {
    float ph = out.isFloor ? (v.viewZ - gh[g]) : (gh[g] - v.viewZ);
    float perp = ph * 192.0f / den;
    float cd = perp / r.cc;
    if (!(ph > 0) || !isfinite(cd) || !(cd > 0)) continue;
    if (cd > best) break;
    float px = v.x + r.rc * cd, py = v.y + r.rs * cd;
#pragma unroll 1
    for (int k = goff[g]; k < goff[g + 1]; ++k) {
      int s = gsec[k];
      if (cd == best && s > out.sector) break;
      if (gd_point_in_sector(sc, s, px, py)) { best = cd; out.sector = s; break; }
    }
  }
  out.unresolved = !isfinite(best);
  return out;
}

/* Pass over the queued pixels.
 *   A  one thread per queued pixel probes it; a resolved pixel is drawn at
 *      once and leaves the queue.
 *   B  only when unresolved pixels remain, once per lane: over the rows of
 *      every pixel that is still unclaimed, one thread per column first looks
 *      below the last of those rows for the nearest resolved row, then sweeps
 *      the rows bottom-up carrying the nearest resolved row below.  It writes
 *      the vertically repaired sector of every pixel of those rows to `vsec`
 *      and one bit per pixel telling whether it anchors horizontal spans.
 *   C  one thread per remaining queued pixel: its own repaired sector, or the
 *      one its nearest anchors left and right agree on. */
__device__ void gd_fallback_pass(const GdScene &sc, const GdView &v, const GdShared &sh, int currentSector,
                                 unsigned short *vsec, bool &sweepDone) {
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int count = min(sh.misc[1], GD_FALLBACK_MAX);
  int *queue = (int *)sh.hitD;
  unsigned *anchors = (unsigned *)sh.hitA;           /* [row][GD_WARPS] column bits */
  unsigned *owned = sh.masks + 7 * GD_SW;            /* drawn pixels are marked owned */
  if (tid == 0) { sh.misc[2] = GD_VH; sh.misc[3] = -1; sh.misc[11] = 0; }
  if (warp == 0) gd_flat_bounds_setup(sc, v, sh.misc);
  __syncthreads();
  const GdFlatBounds b = gd_flat_bounds_load(sh.misc);
  for (int i = tid; i < count; i += GD_THREADS) {
    const int px = queue[i] & 0xFFFF, py = queue[i] >> 16;
    const GdFlatRay r = gd_flat_ray(sc, v, px);
    GdFlatProbe own = gd_flat_probe(sc, v, r, b, py, currentSector);
    if (!own.unresolved) {
      GdPlaneSpan p;
      gd_plane_setup(sc, sh.planeTab, own.sector, own.isFloor, px, p);
      sh.frame[py * GD_SW + px] = gd_plane_pixel(p, v, sh.yslope, sh.colormap, py);
      atomicOr(&owned[(py >> 5) * GD_SW + px], 1u << (py & 31));
      queue[i] = -1;
    } else {
      sh.misc[11] = 1;
    }
  }
  __syncthreads();
  if (sh.misc[11] == 0) return;                       /* block-uniform: nothing unresolved */
  if (!sweepDone) {
    {
      const unsigned *filled = sh.masks + tid, *own = owned + tid;
      int lo = GD_VH, hi = -1;
      for (int k = 0; k < 7; ++k) {
        unsigned m = gd_range_word(k, 0, GD_VH) & ~filled[k * GD_SW] & ~own[k * GD_SW];
        if (m) { lo = min(lo, (k << 5) + __ffs(m) - 1); hi = max(hi, (k << 5) + 31 - __clz(m)); }
      }
      if (hi >= 0) { atomicMin(&sh.misc[2], lo); atomicMax(&sh.misc[3], hi); }
    }
    __syncthreads();
    const int minY = sh.misc[2], maxY = sh.misc[3];
    const GdFlatRay r = gd_flat_ray(sc, v, tid);
    const int flipRow = gd_clamp((int)floorf(r.center) + 1, 0, GD_VH);   /* first floor row */
    /* nearest resolved row below maxY, of maxY's orientation */
    bool haveBelow = false, belowFloor = false;
    int belowSector = 0;
    const int limit = maxY < flipRow ? flipRow : GD_VH;
#pragma unroll 1
    for (int y = maxY + 1; y < limit; ++y) {
      GdFlatProbe q = gd_flat_probe(sc, v, r, b, y, currentSector);
      if (!q.unresolved) { haveBelow = true; belowFloor = q.isFloor; belowSector = q.sector; break; }
    }
    __syncwarp();
#pragma unroll 1
    for (int y = maxY; y >= minY; --y) {
      GdFlatProbe q = gd_flat_probe(sc, v, r, b, y, currentSector);
      bool anchor;
      int repaired;
      if (!q.unresolved) {
        anchor = true;
        repaired = q.sector;
        haveBelow = true; belowFloor = q.isFloor; belowSector = q.sector;
      } else {
        bool spans = haveBelow && belowFloor == q.isFloor;
        repaired = spans ? belowSector : currentSector;
        anchor = spans && belowSector != currentSector;
      }
      vsec[y * GD_SW + tid] = (unsigned short)repaired;
      unsigned m = __ballot_sync(0xffffffffu, anchor);
      if (lane == 0) anchors[y * GD_WARPS + warp] = m;
    }
    sweepDone = true;
    __threadfence_block();
    __syncthreads();
  }
  for (int i = tid; i < count; i += GD_THREADS) {
    if (queue[i] < 0) continue;
    const int px = queue[i] & 0xFFFF, py = queue[i] >> 16;
    int sector = vsec[py * GD_SW + px];
    /* nearest anchor at or left of px, at or right of px */
    int left = -1, right = -1;
#pragma unroll 1
    for (int w = 0; w < GD_WARPS; ++w) {
      unsigned bits = anchors[py * GD_WARPS + w];
      int base = w * 32;
      if (base <= px) {
        unsigned lo = px - base >= 31 ? bits : (bits & ((2u << (px - base)) - 1u));
        if (lo) left = base + 31 - __clz(lo);
      }
      if (base + 31 >= px && right < 0) {
        unsigned hi = px - base <= 0 ? bits : (bits & ~((1u << (px - base)) - 1u));
        if (hi) right = base + __ffs(hi) - 1;
      }
    }
    if (left >= 0 && right >= 0) {
      int sl = vsec[py * GD_SW + left], sr = vsec[py * GD_SW + right];
      if (sl == sr) sector = sl;
    }
    const bool isFloor = ((float)py - gd_flat_ray(sc, v, px).center) > 0;
    GdPlaneSpan p;
    gd_plane_setup(sc, sh.planeTab, sector, isFloor, px, p);
    sh.frame[py * GD_SW + px] = gd_plane_pixel(p, v, sh.yslope, sh.colormap, py);
    atomicOr(&owned[(py >> 5) * GD_SW + px], 1u << (py & 31));
  }
  __syncthreads();
}

/* ---- phase: sprites (engine.py:14138-14228, 14684-14947) ----------------- */
__device__ __noinline__ void gd_actor_setup(const GdScene &sc, const GdView &v, const gd_thing &t, int sector,
                                            GdActor &ac) {
  ac.alive = (t.flags & GD_THING_ALIVE) != 0;
  ac.style = t.style;
  ac.x = t.x; ac.y = t.y;
  int sprite = t.sprite < sc.P ? t.sprite : 0;
  ac.sprite = sprite;
  const int4 si = *reinterpret_cast<const int4 *>(&sc.sprInfo[sprite * 4]);
  ac.w = si.x; ac.h = si.y;
  float dx = t.x - v.x, dy = t.y - v.y;
  float dist = sqrtf(dx * dx + dy * dy);
  if (dist < 1.0f) dist = 1.0f;
  float rel = gd_wrap_angle(atan2f(dy, dx) - v.angle);
  ac.depth = dist * cosf(rel);
  i64 ax = gd_rint(t.x * 65536.0f), ay = gd_rint(t.y * 65536.0f);
  i64 rx = ax - v.vx, ry = ay - v.vy;
  i64 depthFixed = (rx * v.vcos + ry * v.vsin) >> 20;
  i64 sideFixed = (rx * v.vsin - ry * v.vcos) >> 16;
  ac.depthFixed = depthFixed;
  i64 xscale = gd_div(GD_FOCAL_X << 12, gd_max(depthFixed, GD_SPRITE_MIN_DEPTH));
  i64 leftFixed = sideFixed - (i64)si.z * GD_FU;
  i64 left = 160 + (gd_wmul(leftFixed, xscale) >> 32);
  i64 rightFixed = leftFixed + (i64)si.x * GD_FU;
  i64 right = 160 + (gd_wmul(rightFixed, xscale) >> 32);
  ac.xstep = gd_div((i64)si.x << 16, gd_max(right - left, 1));
  ac.left = (int)gd_clamp(left, -(1 << 30), 1 << 30);
  ac.right = (int)gd_clamp(right, -(1 << 30), 1 << 30);
  ac.yscale = gd_div(GD_FOCAL_Y << 12, gd_max(depthFixed, GD_SPRITE_MIN_DEPTH));
  ac.texMid = (i64)si.w * GD_FU - gd_rint((v.viewZ - t.z) * 65536.0f);
  ac.topFixed = v.center - (gd_wmul(ac.texMid, ac.yscale) >> 16);
  ac.iscale = gd_div(GD_U32MASK, gd_max(ac.yscale, 1));
  i64 light = sc.secI[sector * 4] + v.flashLight * 16;
  if (t.flags & GD_THING_BRIGHT) light = 255;
  float base = 61.0f - (float)light / 4.0f;
  float visf = fminf(1280.0f / fmaxf(ac.depth, 1.0f), 24.0f);
  ac.shade = (short)gd_clamp((i64)floorf(base - visf), 0, 31);
}

__device__ __forceinline__ bool gd_behind(const GdScene &sc, const GdWall &wv, int w, const GdActor &ac) {
  i64 nearD = gd_min(wv.dl, wv.dr), farD = gd_max(wv.dl, wv.dr);
  const float4 g = *reinterpret_cast<const float4 *>(&sc.walls[w * 4]);
  float dx = g.z - g.x, dy = g.w - g.y;
  float side = dx * (ac.y - g.y) - dy * (ac.x - g.x);
  return (nearD > ac.depthFixed) || ((farD > ac.depthFixed) && (side <= 0));
}

/* Sprites cluster in a few screen columns, so the drawing is spread by rows:
 * every column thread first lists its visible candidates; then the warps take
 * the listed columns from a counter and draw each candidate's rows 32 at a
 * time, far to near. */
__device__ void gd_sprites(const GdScene &sc, const GdView &v, const GdShared &sh, const GdEvent *events,
                           const int *eventCount, int nThings) {
  const int x0 = threadIdx.x, lane = threadIdx.x & 31;
  if (nThings <= 0) return;                          /* block-uniform */
  unsigned long long *candOf = (unsigned long long *)sh.hitD;       /* per column */
  short *list = (short *)sh.hitA;
  int *counters = &sh.misc[2];                       /* [0] listed columns, [1] next to draw */
  if (x0 == 0) { counters[0] = 0; counters[1] = 0; }
  __syncthreads();
  {
    unsigned long long cand = 0;
    int bw = sh.blockingWall[x0];
    const GdWall &bwv = sh.walls[bw];
    bool bowns = x0 >= bwv.sl && x0 < bwv.sr;
    float wd = sh.wallDistance[x0];
    for (int a = 0; a < nThings; ++a) {
      const GdActor &ac = sh.actors[a];
      if (!(ac.alive && x0 >= ac.left && x0 < ac.right && ac.depth > 0)) continue;
      bool rayVisible = ac.depth < wd;
      rayVisible = rayVisible || !bowns || gd_behind(sc, bwv, bw, ac);
      if (rayVisible) cand |= 1ull << a;
    }
    candOf[x0] = cand;
    if (cand) list[atomicAdd(&counters[0], 1)] = (short)x0;
  }
  __syncthreads();
  const int listed = counters[0];
  for (;;) {
    int slot = 0;
    if (lane == 0) slot = atomicAdd(&counters[1], 1);
    slot = __shfl_sync(0xffffffffu, slot, 0);
    if (slot >= listed) break;
    const int x = list[slot];
    unsigned long long cand = candOf[x];
    const int nEv = eventCount[x];
    const float rayAngle = v.angle + sc.rayOffsets[x];
    const float rayCos = cosf(rayAngle), raySin = sinf(rayAngle);
    /* far to near: repeatedly take the remaining candidate with the largest
     * (depth, index) key */
    while (cand) {
      int pick = -1;
      float pd = 0.0f;
      unsigned long long m = cand;
      while (m) {
        int a = __ffsll((long long)m) - 1;
        m &= m - 1;
        float d = sh.actors[a].depth;
        if (pick < 0 || d >= pd) { pick = a; pd = d; }
      }
      cand &= ~(1ull << pick);
      const GdActor &ac = sh.actors[pick];
      i64 u = (((i64)x - ac.left) * ac.xstep) >> 16;
      if (u < 0 || u >= ac.w) continue;
      const uint8_t *cm = sh.colormap + ac.shade * 256;
      i64 fracBase = ac.texMid - (gd_wmul(v.center - GD_FU, ac.iscale) >> 16);
      /* rows whose source row lies inside the patch */
      int y0 = 0, y1 = GD_VH;
      if (ac.iscale > 0) {
        /* frac(y) >> 16 in [0,h)  <=>  0 <= fracBase + y*iscale < h*FU */
        i64 lo = -fracBase, hi = (i64)ac.h * GD_FU - fracBase;
        i64 ya = lo <= 0 ? 0 : gd_div(lo + ac.iscale - 1, ac.iscale);
        i64 yb = hi <= 0 ? 0 : gd_div(hi + ac.iscale - 1, ac.iscale);
        y0 = (int)gd_clamp(ya, 0, GD_VH);
        y1 = (int)gd_clamp(yb, 0, GD_VH);
      }
      __syncwarp();                                  /* the farther sprite's pixels are in place */
#pragma unroll 1
      for (int y = y0 + lane; y < y1; y += 32) {
        i64 frac = fracBase + (i64)y * ac.iscale;
        i64 tv = frac >> 16;
        if (tv < 0 || tv >= ac.h) continue;
        size_t si = ((size_t)ac.sprite * sc.sprH + (size_t)tv) * sc.sprW + (size_t)u;
        uint8_t post = sc.sprPost[si];
        if (post == 255) continue;
        i64 postTop = (ac.topFixed + ac.yscale * (i64)post) >> 16;
        if (y < postTop) continue;
        /* nearest clip event covering this pixel */
        float bestD = GD_INF;
        int bestW = -1, ownerSector = -1;
        bool filled = false, ownerFloor = false;
#pragma unroll 1
        for (int e = 0; e < nEv; ++e) {
          const GdEvent ev = events[e * GD_SW + x];
          bool inLower = y >= ev.t1a && y < ev.t1b, inUpper = y >= ev.t0a && y < ev.t0b;
          bool drawn = inLower ? ((ev.pad0 & 2) != 0) : (inUpper ? ((ev.pad0 & 1) != 0) : false);
          bool covers = (y < ev.silTop) || (y >= ev.silBot);
          if (drawn && !filled) { filled = true; covers = true; }
          if (covers && ev.dist < bestD) { bestD = ev.dist; bestW = ev.wall; }
          if (ownerSector < 0 && ev.sector >= 0) {
            if (y >= ev.floorA && y < ev.floorB) { ownerSector = ev.sector; ownerFloor = true; }
            else if (y >= ev.ceilA && y < ev.ceilB) ownerSector = ev.sector;
          }
        }
        bool visible;
        if (bestW >= 0) {
          visible = gd_behind(sc, sh.walls[bestW], bestW, ac);
        } else {
          float limit = GD_INF;
          if (!filled && ownerSector >= 0 && gd_pixel_unresolved(sc, v, x, y, rayCos, raySin, ownerSector))
            limit = gd_plane_depth(sc, v, ownerSector, ownerFloor, y);
          visible = ac.depth < limit;
        }
        if (!visible) continue;
        uint8_t lit = cm[sc.sprAtlas[si]];
        uint8_t dst = sh.frame[y * GD_SW + x];
        uint8_t out = lit;
        if (ac.style == -2) out = sc.transLut[dst * 256 + lit];
        else if (ac.style >= 0) out = sc.addLut[((ac.style > 1 ? 1 : ac.style) * 256 + dst) * 256 + lit];
        sh.frame[y * GD_SW + x] = out;
      }
    }
    __syncwarp();
  }
}

/* ---- phase: weapon (engine.py:14994-15121) ------------------------------ */
__device__ __noinline__ void gd_weapon_patch(const GdScene &sc, uint8_t *frame, int id, i64 hoff, i64 voff) {
  if (id < 0 || id >= sc.Q) return;
  const int4 wi = *reinterpret_cast<const int4 *>(&sc.wpnInfo[id * 4]);
  int w = wi.x, h = wi.y;
  if (w <= 0 || h <= 0) return;
  i64 screenLeft = (hoff - (i64)wi.z * GD_FU) >> 16;
  i64 texMid = 100 * GD_FU - (32 * GD_FU + 0x6000) - voff + (i64)wi.w * GD_FU;
  const i64 yscale = GD_SCREEN_H * GD_FU / 200;
  const i64 iscale = GD_U32MASK / yscale;
  /* rows whose source row lies inside the patch: 0 <= base + y*iscale < h*FU */
  const i64 base = texMid - (i64)(GD_VH / 2 - 1) * iscale;
  const i64 lo = -base, hi = (i64)h * GD_FU - base;
  const int y0 = (int)gd_clamp(lo <= 0 ? 0 : gd_div(lo + iscale - 1, iscale), 0, GD_VH);
  const int y1 = (int)gd_clamp(hi <= 0 ? 0 : gd_div(hi + iscale - 1, iscale), 0, GD_VH);
  for (int idx = threadIdx.x; idx < (y1 - y0) * w; idx += GD_THREADS) {
    int y = y0 + idx / w, sx = idx - (y - y0) * w;
    i64 xx = screenLeft + sx;
    if (xx < 0 || xx >= GD_SW) continue;
    i64 sy = (base + (i64)y * iscale) >> 16;
    if (sy < 0 || sy >= h) continue;
    i64 cy = gd_min(sy, sc.wpnH - 1), cx = gd_min((i64)sx, (i64)sc.wpnW - 1);
    size_t si = ((size_t)id * sc.wpnH + (size_t)cy) * sc.wpnW + (size_t)cx;
    if (sc.wpnOpaque[si]) frame[y * GD_SW + (int)xx] = sc.wpnAtlas[si];
  }
}

__device__ void gd_weapon(const GdScene &sc, const int32_t *lane, uint8_t *frame) {
  if (!sc.wpnAvailable) return;
  if (lane[GD_L_FLAGS] & 1) return;
  int weapon = (int)gd_clamp(lane[GD_L_WEAPON], 0, 7);
  int cooldown = (int)gd_clamp(lane[GD_L_WPN_COOLDOWN], 0, sc.wpnTics - 1);
  int parity = (int)gd_pymod(lane[GD_L_WPN_FIRE_COUNT], 2);
  if (weapon == 1 && cooldown == 0) parity = (int)gd_pymod(gd_max(lane[GD_L_WPN_READY_TICS] - 1, 0) / 4, 2);
  int ti = (weapon * 2 + parity) * sc.wpnTics + cooldown;
  int frameId = sc.wpnFrameIds[ti], flashId = sc.wpnFlashIds[ti];
  i64 lowerTics = gd_clamp(16 - (i64)lane[GD_L_WPN_LOWER], 0, 16);
  i64 verticalTics = lane[GD_L_WPN_PENDING] >= 0 ? lowerTics : (i64)lane[GD_L_WPN_RAISE];
  i64 spawnRaise = gd_clamp(14 - ((i64)lane[GD_L_EPISODE_TIME] - 1), 0, 14);
  verticalTics = gd_max(verticalTics, spawnRaise);
  bool ready = lane[GD_L_WPN_COOLDOWN] <= 0 && lane[GD_L_WPN_RAISE] <= 0 && lane[GD_L_WPN_PENDING] < 0;
  i64 bobAngle = ((i64)lane[GD_L_EPISODE_TIME] * 128) & 8191;
  i64 bob = lane[GD_L_BOB_FIXED];
  i64 bobx = (bob * sc.fineSine[(bobAngle + 2048) & 8191]) >> 16;
  i64 boby = (bob * sc.fineSine[bobAngle & 4095]) >> 16;
  if (!ready) { bobx = 0; boby = 0; }
  i64 voff = verticalTics * 6 * GD_FU + boby;
  gd_weapon_patch(sc, frame, frameId, bobx, voff);
  __syncthreads();
  if (flashId >= 0) gd_weapon_patch(sc, frame, flashId, bobx, voff);
}

/* ---- phase: status bar (engine.py:15158-15267) --------------------------- */
/* The status bar is a list of up to GD_HUD_MAX_PATCHES opaque-masked blits drawn
 * in a fixed order, later ones on top.  Thread 0 lists (patch, x, y), one thread
 * per entry clips it against the canvas, and then every column thread resolves
 * its 32 pixels from the entries that cross its column, topmost first. */
#define GD_HUD_MAX_PATCHES 48

struct GdHudList { int4 *entries; int *count; };

__device__ __forceinline__ void gd_hud_push(const GdHudList &hl, int patch, int x, int y) {
  int n = *hl.count;
  if (n < GD_HUD_MAX_PATCHES) { hl.entries[n] = make_int4(patch, x, y, 0); *hl.count = n + 1; }
}

__device__ void gd_hud_number(const GdScene &sc, const GdHudList &hl, int value, int right, int y, bool small) {
  int vc = value < -99 ? -99 : (value > 999 ? 999 : value);
  int neg = vc < 0;
  int mag = neg ? -vc : vc;
  int digits[3], n = 0;
  do { digits[n++] = mag % 10; mag /= 10; } while (mag > 0);
  int len = n + neg;
  int dw = small ? 4 : 14, base = small ? 28 : 2;
  int x = right - len * dw;
  if (neg) x += dw;
  for (int k = n - 1; k >= 0; --k) {
    int patch = base + digits[k];
    const int4 hi = *reinterpret_cast<const int4 *>(&sc.hudInfo[patch * 4]);
    gd_hud_push(hl, patch, x - hi.z, y - hi.w);   /* the blit subtracts the glyph offsets once more */
    x += dw;
  }
}

__device__ __noinline__ void gd_hud(const GdScene &sc, const GdShared &sh, const int32_t *lane, uint8_t *canvas) {
  GdHudList hl;
  hl.entries = (int4 *)sh.obs;                       /* free until the resize */
  hl.count = (int *)(sh.obs + GD_HUD_MAX_PATCHES * sizeof(int4));
  if (threadIdx.x == 0) {
    *hl.count = 0;
    gd_hud_push(hl, 0, 0, 0);
    gd_hud_push(hl, 1, 104, 0);
    int weapon = lane[GD_L_WEAPON];
    int ammoSlot = weapon < 2 ? -1 : (int)((0x54122100u >> (4 * (weapon > 7 ? 7 : weapon))) & 0xF);   /* -,-,1,2,2,1,4,5 */
    int ammo = ammoSlot < 0 ? 0 : (int)__int_as_float(lane[GD_L_READY_AMMO]);
    float hf = __int_as_float(lane[GD_L_HEALTH]), af = __int_as_float(lane[GD_L_ARMOR]);
    int health = (int)(hf < 0 ? 0.0f : (hf > 999 ? 999.0f : hf));
    int armor = (int)(af < 0 ? 0.0f : (af > 999 ? 999.0f : af));
    gd_hud_number(sc, hl, ammo, 44, 3, false);
    gd_hud_number(sc, hl, health, 90, 3, false);
    gd_hud_push(hl, 12, 90, 3);
    gd_hud_number(sc, hl, armor, 221, 3, false);
    gd_hud_push(hl, 12, 221, 3);
    int pain = (100 - health) >= 0 ? (100 - health) / 20 : -((health - 100 + 19) / 20);
    pain = pain < 0 ? 0 : (pain > 4 ? 4 : pain);
    int face = 13 + pain * 3 + lane[GD_L_FACE_INDEX];
    if (lane[GD_L_GRIN_TICS] > 0) face = 64 + pain;
    else if (lane[GD_L_PAIN_TICS] > 0) {
      if (lane[GD_L_FLAGS] & 2) face = 59 + pain;
      else {
        int d = lane[GD_L_PAIN_DIRECTION];
        d = d < 0 ? 0 : (d > 2 ? 2 : d);
        face = (d == 0 ? 44 : (d == 1 ? 49 : 54)) + pain;
      }
    } else if (lane[GD_L_ATTACK_HELD] >= 70) face = 49 + pain;
    if (health <= 0) face = 69;
    gd_hud_push(hl, face < 0 ? 0 : (face > 69 ? 69 : face), 143, 0);
    for (int wi = 0; wi < 6; ++wi) {
      bool owned = wi < 5 && ((lane[GD_L_WEAPONS_OWNED] >> (wi + 1)) & 1);
      gd_hud_push(hl, owned ? 28 + wi + 2 : 38 + wi, 111 + 12 * (wi % 3), wi < 3 ? 4 : 14);
    }
    for (int row = 0; row < 4; ++row) {
      int y = 5 + row * 6;
      gd_hud_number(sc, hl, (int)__int_as_float(lane[GD_L_AMMO0 + row]), 288, y, true);
      gd_hud_number(sc, hl, row == 0 ? 200 : (row == 3 ? 300 : 50), 314, y, true);   /* ammo maxima */
    }
  }
  __syncthreads();
  const int n = *hl.count;
  if (threadIdx.x < n) {
    /* clip against the canvas: (tx | ty << 16, cw | ch << 16, sx | sy << 16, patch); cw = 0 when nothing is left */
    int4 e = hl.entries[threadIdx.x];
    const int patch = e.x;
    const int4 hi = *reinterpret_cast<const int4 *>(&sc.hudInfo[patch * 4]);
    int x = e.y - hi.z, y = e.z - hi.w;
    int w = hi.x, h = hi.y;
    int sx = x < 0 ? -x : 0, sy = y < 0 ? -y : 0;
    int tx = x > 0 ? x : 0, ty = y > 0 ? y : 0;
    int cw = min(w - sx, GD_SW - tx), ch = min(h - sy, GD_HUD_H - ty);
    if (w <= 0 || h <= 0 || cw <= 0 || ch <= 0) { cw = 0; ch = 0; }
    hl.entries[threadIdx.x] = make_int4(tx | (ty << 16), cw | (ch << 16), sx | (sy << 16), patch);
  }
  __syncthreads();
  {
    const int x = threadIdx.x;
    unsigned long long mine = 0;                       /* entries that cross this column */
    for (int k = 0; k < n; ++k) {
      int4 e = hl.entries[k];
      int tx = e.x & 0xFFFF, cw = e.y & 0xFFFF;
      if (x >= tx && x < tx + cw) mine |= 1ull << k;
    }
    for (int y = 0; y < GD_HUD_H; ++y) {
      uint8_t value = 0;
      unsigned long long m = mine;
      while (m) {
        int k = 63 - __clzll((long long)m);            /* topmost remaining entry */
        m &= ~(1ull << k);
        int4 e = hl.entries[k];
        int tx = e.x & 0xFFFF, ty = e.x >> 16, ch = e.y >> 16, sx = e.z & 0xFFFF, sy = e.z >> 16;
        if (y < ty || y >= ty + ch) continue;
        size_t si = ((size_t)e.w * GD_HUD_H + (size_t)(sy + y - ty)) * GD_SW + (size_t)(sx + x - tx);
        if (sc.hudOpaque[si]) { value = sc.hudAtlas[si]; break; }
      }
      canvas[y * GD_SW + x] = value;
    }
  }
  __syncthreads();
}

/* ---- phase: 320x240 -> 84x84 area resize + grayscale ---------------------
 * Integer definition: src/gradoom/_triton_kernels.py:120-177.  The weights
 * (y_overlap*x_overlap)/48 factor exactly into (y_overlap/12)*(x_overlap/4). */
__device__ void gd_resize(const uint8_t *frame, const unsigned long long *pal64, int srcRows, uint8_t *out) {
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
      const uint8_t *row = frame + min(sy, GD_SCREEN_H - 1) * GD_SW;
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

/* ---- the kernel ----------------------------------------------------------- */
extern __shared__ __align__(16) uint8_t gd_smem[];

__global__ void __launch_bounds__(GD_THREADS, 1) gd_render_kernel(const GdParams p) {
  /* The scene descriptor, the shared-memory map and the lane's view are read by
   * every helper through references; keeping them in shared memory (one copy
   * per CTA) keeps those reads off the per-thread stack. */
  __shared__ GdScene sScene;
  __shared__ GdShared sShared;
  __shared__ GdView sView;
  const int tid = threadIdx.x;
  GdRowProj *stagedRowproj = nullptr;
  {
    GdScene sc = p.sc;
    GdShared sh;
    gd_carve(gd_smem, sc.W, p.maxThings, sh);
    uint8_t *cursor = gd_smem + gd_shared_bytes(sc.W, p.maxThings);
    const int m = p.stageMask;
    if (m & GD_STAGE_WALLS) sc.walls = (const float *)gd_stage_copy(cursor, sc.walls, (size_t)sc.W * 16);
    if (m & GD_STAGE_WSEC) sc.wsec = (const int32_t *)gd_stage_copy(cursor, sc.wsec, (size_t)sc.W * 8);
    if (m & GD_STAGE_SECLIST) {
      sc.secOff = (const int32_t *)gd_stage_copy(cursor, sc.secOff, (size_t)(sc.S + 1) * 4);
      sc.secWalls = (const int32_t *)gd_stage_copy(cursor, sc.secWalls, (size_t)(p.secWallsN > 0 ? p.secWallsN : 1) * 4);
    }
    if (m & GD_STAGE_SECTORS) {
      sc.secF = (const float *)gd_stage_copy(cursor, sc.secF, (size_t)sc.S * 8);
      sc.secI = (const int32_t *)gd_stage_copy(cursor, sc.secI, (size_t)sc.S * 16);
    }
    if (m & GD_STAGE_WVTX) sc.wvtx = (const int32_t *)gd_stage_copy(cursor, sc.wvtx, (size_t)sc.W * 8);
    if (m & GD_STAGE_WLEN) sc.wlen = (const float *)gd_stage_copy(cursor, sc.wlen, (size_t)sc.W * 4);
    if (m & GD_STAGE_SIDETEX) sc.sideTex = (const int32_t *)gd_stage_copy(cursor, sc.sideTex, (size_t)sc.W * 24);
    if (m & GD_STAGE_SIDEOFF) sc.sideOff = (const float *)gd_stage_copy(cursor, sc.sideOff, (size_t)sc.W * 16);
    if (m & GD_STAGE_VTXLIST) {
      sc.vtxOff = (const int32_t *)gd_stage_copy(cursor, sc.vtxOff, (size_t)(p.V + 1) * 4);
      sc.vtxWalls = (const int32_t *)gd_stage_copy(cursor, sc.vtxWalls, (size_t)(p.vtxWallsN > 0 ? p.vtxWallsN : 1) * 4);
    }
    if (m & GD_STAGE_ROWPROJ) { stagedRowproj = (GdRowProj *)cursor; cursor += gd_align16((size_t)sc.W * 4 * sizeof(GdRowProj)); }
    sh.planeTab = (GdPlaneEntry *)(p.scratch + (size_t)blockIdx.x * gd_scratch_per_cta(sc.W, sc.S) + GD_SCRATCH_FIXED);
    if (tid == 0) { sScene = sc; sShared = sh; }
  }
  __syncthreads();
  const GdScene &sc = sScene;
  const GdShared &sh = sShared;
  /* tables shared by every lane this CTA draws */
  for (int i = tid; i < 32 * 256 / 4; i += GD_THREADS)
    ((unsigned *)sh.colormap)[i] = ((const unsigned *)sc.colormap)[i];
  gd_lane_palette(sc, sh, 0);
  bool paletteBlended = false;    /* CTA-uniform: the shared palette holds a lane's screen-flash blend */
  uint8_t *myScratch = p.scratch + (size_t)blockIdx.x * gd_scratch_per_cta(sc.W, sc.S);
  GdEvent *events = (GdEvent *)myScratch;
  int *eventCount = (int *)(myScratch + GD_SCRATCH_EVENTS_BYTES);
  unsigned short *vsec = (unsigned short *)(myScratch + GD_SCRATCH_EVENTS_BYTES + GD_SW * 4);
  GdRowProj *rowproj = stagedRowproj ? stagedRowproj
                                     : (GdRowProj *)(myScratch + GD_SCRATCH_FIXED + gd_scratch_plane_bytes(sc.S));

#ifdef GD_PROFILE_PHASES
  if (tid == 0 && blockIdx.x == 0) gdProfile = (unsigned long long *)(p.status + 8);
  long long gdT0 = clock64();
  const long long gdStartClock = gdT0;
  unsigned long long gdStartNs;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(gdStartNs));
#define GD_BEAT(ph) do { __syncthreads(); if (tid == 0) { long long t = clock64(); atomicAdd((unsigned long long *)(p.status + 8) + (ph), (unsigned long long)(t - gdT0)); gdT0 = t; } } while (0)
#else
#define GD_BEAT(ph) do {} while (0)
#endif
  /* Lanes differ a lot in cost (a long corridor crosses many sectors), so the
   * persistent CTAs take lanes from a shared counter instead of a fixed stride.
   * The counter pair lives behind the event scratch and is left at zero by the
   * last CTA to finish. */
  unsigned *queue = (unsigned *)(p.scratch + (size_t)p.queueOffset);
  __shared__ int nextLane;
  for (;;) {
    __syncthreads();
    if (tid == 0) nextLane = (int)atomicAdd(&queue[0], 1u);
    __syncthreads();
    const int l = nextLane;
    if (l >= p.n) break;
    GD_BEAT(1);
    if (p.flags & GD_F_STACK_FILL) {
      if (p.resetMask && !p.resetMask[l]) continue;  /* uniform across the CTA */
    }
    if (tid < GD_LANE_WORDS) sh.lane[tid] = p.lanes[(size_t)l * GD_LANE_WORDS + tid];
    if (tid < 10) sh.ownerMask[tid] = 0;
    if (tid == 0) sh.misc[1] = 0;
    /* sector of every thing and of the player (slot 64): lowest index that
     * contains the point (engine.py:9598-9617), found by all threads together
     * while thread 0 sets up the view */
    int *pointSector = (int *)sh.hitA;
    if (tid <= 64) pointSector[tid] = 0x7fffffff;
    __syncthreads();
    {
      const int laneFlags = sh.lane[GD_L_FLAGS];
      const bool wantBlend = (laneFlags & 4) != 0;
      if (wantBlend || paletteBlended) gd_lane_palette(sc, sh, laneFlags);   /* read again after later barriers */
      paletteBlended = wantBlend;
    }
    int nThings = sh.lane[GD_L_THINGS];
    if (nThings > p.maxThings || nThings > 64) {
      if (tid == 0) atomicOr(p.status, GD_STATUS_THINGS_OVERFLOW);
      nThings = min(p.maxThings, 64);
    }
    if (nThings < 0) nThings = 0;
    if (tid == 0) {
      gd_view_setup(sc, sh.lane, sView);
    } else if (tid >= 32) {
      const int pairs = (nThings + 1) * sc.S;
      for (int i = tid - 32; i < pairs; i += GD_THREADS - 32) {
        int t = i / sc.S, s = i - t * sc.S;
        float px, py;
        if (t < nThings) {
          const gd_thing &th = p.things[(size_t)l * p.maxThings + t];
          px = th.x; py = th.y;
        } else {
          px = __int_as_float(sh.lane[GD_L_X]); py = __int_as_float(sh.lane[GD_L_Y]);
          t = 64;
        }
        if (gd_point_in_sector(sc, s, px, py)) atomicMin(&pointSector[t], s);
      }
    }
    __syncthreads();
    const GdView &v = sView;
    if (tid < GD_VH) {
      /* yslope of the row (engine.py:10933-10946) */
      i64 centerRow = v.center >> 16;
      i64 den = (tid < centerRow) ? (v.center - (i64)tid * GD_FU - GD_FU / 2) : ((i64)tid * GD_FU - v.center + GD_FU / 2);
      den = gd_max(den, 1);
      i64 ys = gd_div(GD_FOCAL_Y << 16, den);
      if (den <= (GD_FOCAL_Y >> 15)) ys = (1LL << 31) - 1;
      sh.yslope[tid] = (unsigned)ys;
    }
    for (int w = tid; w < sc.W; w += GD_THREADS) gd_project_wall(sc, v, w, sh.walls[w]);
    for (int idx = GD_THREADS - 1 - tid; idx < sc.S * 2; idx += GD_THREADS)   /* the threads the walls leave idle */
      gd_plane_entry_setup(sc, v, idx >> 1, (idx & 1) != 0, sh.planeTab[idx]);
    for (int a = tid; a < nThings; a += GD_THREADS) {
      int sector = pointSector[a] == 0x7fffffff ? 0 : pointSector[a];
      gd_actor_setup(sc, v, p.things[(size_t)l * p.maxThings + a], sector, sh.actors[a]);
    }
    if (tid == GD_THREADS - 1) sh.misc[0] = pointSector[64] == 0x7fffffff ? 0 : pointSector[64];
    __syncthreads();
    GD_BEAT(2);
    gd_wall_spans(sc, v, sh);
    /* row projection tables, for the walls that passed the frustum test (the
     * walk selects no other wall) */
    for (int idx = tid; idx < sh.misc[2] * 4; idx += GD_THREADS) {
      int w = ((const short *)sh.hitD)[idx >> 2], slot = idx & 3;
      int sector = sc.wsec[w * 2 + (slot >> 1)];
      if (sector >= 0) gd_rowproj_setup(v, sh.walls[w], sc.secF[sector * 2 + (slot & 1)], rowproj[w * 4 + slot]);
    }
    __syncthreads();
    GD_BEAT(3);
    const short *frustumList = (const short *)sh.hitD;
    const int frustumListed = sh.misc[2];
    for (int i = tid; i < frustumListed; i += GD_THREADS) {   /* walls outside the frustum own no column */
      const int w = frustumList[i];
      int xl = sh.walls[w].isl;
      if (xl >= 0 && xl < GD_SW) {
        float rx, ry;
        gd_ray(v, xl, rx, ry);
        GdHit h = gd_hit(sc, v, sh.walls, w, xl, rx, ry);
        if (isfinite(h.d)) atomicOr(&sh.ownerMask[xl >> 5], 1u << (xl & 31));
      }
    }
    {
      float rx, ry, wd;
      int bw;
      gd_ray(v, tid, rx, ry);
      gd_blocking_raycast(sc, v, sh, frustumList, frustumListed, rx, ry, wd, bw);
      sh.wallDistance[tid] = wd;
      sh.blockingWall[tid] = (short)bw;
    }
    __syncthreads();
    GD_BEAT(4);
    gd_walk(sc, v, sh, events, eventCount, rowproj, p.status, sh.misc[0]);
    __syncthreads();
    /* Rows no seg ever claimed show the per-pixel flat fallback.  They are
     * queued (the hit cache is free once every column has finished its walk)
     * and resolved; a frame with more such pixels than the queue holds takes
     * several rounds, each pass marking what it drew as owned. */
    bool sweepDone = false;                          /* CTA-uniform */
    for (;;) {
      const unsigned *filled = sh.masks + tid, *owned = sh.masks + 7 * GD_SW + tid;
      for (int k = 0; k < 7; ++k) {
        unsigned m = gd_range_word(k, 0, GD_VH) & ~filled[k * GD_SW] & ~owned[k * GD_SW];
        while (m) {
          int y = (k << 5) + __ffs(m) - 1;
          m &= m - 1;
          int slot = atomicAdd(&sh.misc[1], 1);
          if (slot < GD_FALLBACK_MAX) ((int *)sh.hitD)[slot] = (y << 16) | tid;
        }
      }
      __syncthreads();
      const int queued = sh.misc[1];
      if (queued == 0) break;                        /* block-uniform */
      gd_fallback_pass(sc, v, sh, sh.misc[0], vsec, sweepDone);
      if (queued <= GD_FALLBACK_MAX) break;
      if (tid == 0) sh.misc[1] = 0;
      __syncthreads();
    }
    if (sc.M > 0) {
      gd_masked_pass(sc, v, sh);
      __syncthreads();
    }
    GD_BEAT(5);
    gd_sprites(sc, v, sh, events, eventCount, nThings);
    __syncthreads();
    GD_BEAT(6);
    gd_weapon(sc, sh.lane, sh.frame);
    __syncthreads();
    GD_BEAT(7);
    const bool wantFull = p.indexedOut != nullptr || p.rgbOut != nullptr;
    if (p.flags & GD_F_DRAW_HUD) {
      gd_hud(sc, sh, sh.lane, sh.frame + GD_VH * GD_SW);
    } else if (wantFull) {
      for (int i = tid; i < GD_HUD_H * GD_SW / 4; i += GD_THREADS) ((unsigned *)(sh.frame + GD_VH * GD_SW))[i] = 0;
      __syncthreads();
    }
    if (p.indexedOut) {
      uint4 *dst = (uint4 *)(p.indexedOut + (size_t)l * GD_SCREEN_H * GD_SW);
      const uint4 *src = (const uint4 *)sh.frame;
      for (int i = tid; i < GD_SCREEN_H * GD_SW / 16; i += GD_THREADS) dst[i] = src[i];
    }
    if (p.rgbOut) {
      /* four pixels (one word of indices) become three words of RGB24 */
      unsigned *dst = (unsigned *)(p.rgbOut + (size_t)l * GD_SCREEN_H * GD_SW * 3);
      const unsigned *src = (const unsigned *)sh.frame;
      for (int q = tid; q < GD_SCREEN_H * GD_SW / 4; q += GD_THREADS) {
        const unsigned idx = src[q];
        const unsigned p0 = sh.pal32[idx & 0xFF], p1 = sh.pal32[(idx >> 8) & 0xFF];
        const unsigned p2 = sh.pal32[(idx >> 16) & 0xFF], p3 = sh.pal32[idx >> 24];
        dst[q * 3 + 0] = p0 | (p1 << 24);
        dst[q * 3 + 1] = (p1 >> 8) | (p2 << 16);
        dst[q * 3 + 2] = (p2 >> 16) | (p3 << 8);
      }
    }
    GD_BEAT(8);
    if (p.stack || p.obsOut) {
      int srcRows = (p.flags & GD_F_MASK_HUD) ? GD_VH : GD_SCREEN_H;
      gd_resize(sh.frame, sh.pal64, srcRows, sh.obs);
      __syncthreads();
      const uint4 *src = (const uint4 *)sh.obs;
      const int vecs = GD_OBS * GD_OBS / 16;  /* 441 */
      if (p.obsOut) {
        uint4 *dst = (uint4 *)(p.obsOut + (size_t)l * GD_OBS * GD_OBS);
        for (int i = tid; i < vecs; i += GD_THREADS) dst[i] = src[i];
      }
      if (p.stack) {
        uint4 *s0 = (uint4 *)(p.stack + (size_t)l * GD_STACK * GD_OBS * GD_OBS);
        if (p.flags & GD_F_STACK_FILL) {
          for (int i = tid; i < vecs; i += GD_THREADS) {
            uint4 val = src[i];
            s0[i] = val; s0[vecs + i] = val; s0[2 * vecs + i] = val; s0[3 * vecs + i] = val;
          }
        } else if (p.flags & GD_F_STACK_ROLL) {
          for (int i = tid; i < vecs; i += GD_THREADS) {
            s0[i] = s0[vecs + i];
            s0[vecs + i] = s0[2 * vecs + i];
            s0[2 * vecs + i] = s0[3 * vecs + i];
            s0[3 * vecs + i] = src[i];
          }
        } else {
          for (int i = tid; i < vecs; i += GD_THREADS) s0[3 * vecs + i] = src[i];
        }
      }
    }
  }
#ifdef GD_PROFILE_PHASES
  if (tid == 0) {
    unsigned long long ns;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(ns));
    atomicAdd((unsigned long long *)(p.status + 8) + 12, ns - gdStartNs);
    atomicAdd((unsigned long long *)(p.status + 8) + 13, (unsigned long long)(clock64() - gdStartClock));
  }
#endif
  if (tid == 0) {
    __threadfence();
    if (atomicAdd(&queue[1], 1u) == gridDim.x - 1) {
      queue[0] = 0;
      queue[1] = 0;
      __threadfence();
    }
  }
}

/* ---- C ABI (declared in include/gradoom_b200.h) --------------------------- */
#include "../../include/gradoom_b200.h"

#include <new>
#include <string.h>

#define GD_HOST_CHUNKS 4

struct gd_renderer {
  GdScene sc;
  int32_t header[GD_HDR_WORDS];
  int device;
  int maxThings;
  int ctas;
  size_t smemBytes;
  int stageMask;
  int secWallsN, vtxWallsN, V;
  /* gd_render_step_host overlaps the device->host copy of one lane chunk with
   * the drawing of the next on this side stream */
  cudaStream_t copyStream;
  cudaEvent_t chunkDone[GD_HOST_CHUNKS], copiesDone;
};

static const void *gd_section(const uint8_t *dev, const int32_t *h, int s) { return dev + h[GD_HDR_SECTION0 + s]; }

extern "C" const char *gd_error_string(int code) {
  switch (code) {
    case GD_OK: return "ok";
    case GD_ERR_NULL: return "null pointer argument";
    case GD_ERR_BLOB: return "scene blob has a bad magic, version or size";
    case GD_ERR_UNSUPPORTED: return "scene uses a feature this render path does not draw";
    case GD_ERR_SIZE: return "size argument out of range";
    case GD_ERR_ALIGN: return "device pointer is not 16-byte aligned";
    case GD_ERR_CUDA: return "CUDA runtime call failed";
    case GD_ERR_SCRATCH: return "scratch buffer is too small";
    case GD_ERR_SHARED: return "scene needs more shared memory than one SM offers";
    case GD_ERR_STATIC_LIMIT: return "scene or device index exceeds the limits of the built-in scratch array";
    case GD_ERR_DEVICE: return "the renderer's device is not the current CUDA device";
    default: return "unknown error";
  }
}

extern "C" int gd_renderer_create(const void *blob_header_host, const void *blob_dev, size_t blob_bytes, int device,
                                  int max_things, gd_renderer **out) {
  if (!blob_header_host || !blob_dev || !out) return GD_ERR_NULL;
  if (blob_bytes < GD_HDR_WORDS * 4) return GD_ERR_BLOB;
  if (((uintptr_t)blob_dev) & 15) return GD_ERR_ALIGN;
  if (max_things < 0 || max_things > 64) return GD_ERR_SIZE;
  const int32_t *h = (const int32_t *)blob_header_host;
  if (h[GD_H_MAGIC] != GD_MAGIC || h[GD_H_VERSION] != GD_VERSION || (size_t)h[GD_H_BYTES] != blob_bytes)
    return GD_ERR_BLOB;
  if (h[GD_H_UNSUPPORTED] != 0) return GD_ERR_UNSUPPORTED;
  if (h[GD_H_WALLS] <= 0 || h[GD_H_WALLS] >= 32768 || h[GD_H_SECTORS] <= 0 || h[GD_H_SECTORS] >= 32768)
    return GD_ERR_SIZE;
  gd_renderer *r = new (std::nothrow) gd_renderer;
  if (!r) return GD_ERR_CUDA;
  r->copyStream = nullptr;
  r->copiesDone = nullptr;
  for (int c = 0; c < GD_HOST_CHUNKS; ++c) r->chunkDone[c] = nullptr;
  memcpy(r->header, h, sizeof r->header);
  r->device = device;
  r->maxThings = max_things;
  const uint8_t *d = (const uint8_t *)blob_dev;
  GdScene &sc = r->sc;
  sc.W = h[GD_H_WALLS]; sc.S = h[GD_H_SECTORS]; sc.T = h[GD_H_TEXTURES];
  sc.texH = h[GD_H_TEX_H]; sc.texW = h[GD_H_TEX_W];
  sc.P = h[GD_H_SPRITES]; sc.sprH = h[GD_H_SPR_H]; sc.sprW = h[GD_H_SPR_W];
  sc.Q = h[GD_H_WPN_PATCHES]; sc.wpnH = h[GD_H_WPN_H]; sc.wpnW = h[GD_H_WPN_W]; sc.wpnTics = h[GD_H_WPN_TICS];
  sc.nStarts = h[GD_H_STARTS]; sc.B = h[GD_H_BLOCKING]; sc.nbDirect = h[GD_H_NB_DIRECT];
  sc.wpnAvailable = h[GD_H_WPN_AVAILABLE];
#define SECP(type, name) (const type *)gd_section(d, h, name)
  sc.walls = SECP(float, GD_S_WALLS); sc.wsec = SECP(int32_t, GD_S_WALL_SECTORS); sc.wlen = SECP(float, GD_S_WALL_LEN);
  sc.sideTex = SECP(int32_t, GD_S_SIDE_TEX); sc.sideOff = SECP(float, GD_S_SIDE_OFF);
  sc.wvtx = SECP(int32_t, GD_S_WALL_VTX); sc.vtxOff = SECP(int32_t, GD_S_VTX_OFF); sc.vtxWalls = SECP(int32_t, GD_S_VTX_WALLS);
  sc.nbDirectTab = SECP(int32_t, GD_S_NB_DIRECT); sc.nbOff = SECP(int32_t, GD_S_NB_OFF);
  sc.nbIdx = SECP(int32_t, GD_S_NB_IDX); sc.nbFlags = SECP(int32_t, GD_S_NB_FLAGS);
  sc.sbStartOff = SECP(int32_t, GD_S_SB_START_OFF); sc.sbStartIdx = SECP(int32_t, GD_S_SB_START_IDX);
  sc.sbEndOff = SECP(int32_t, GD_S_SB_END_OFF); sc.sbEndIdx = SECP(int32_t, GD_S_SB_END_IDX);
  sc.secF = SECP(float, GD_S_SECTOR_F); sc.secI = SECP(int32_t, GD_S_SECTOR_I);
  sc.secOff = SECP(int32_t, GD_S_SEC_OFF); sc.secWalls = SECP(int32_t, GD_S_SEC_WALLS);
  sc.edgeOff = SECP(int32_t, GD_S_EDGE_OFF); sc.edgeWalls = SECP(int32_t, GD_S_EDGE_WALLS);
  sc.blocking = SECP(int32_t, GD_S_BLOCKING);
  sc.texInfo = SECP(int32_t, GD_S_TEX_INFO); sc.texAtlas = SECP(uint8_t, GD_S_TEX_ATLAS);
  sc.texAtlasCol = SECP(uint8_t, GD_S_TEX_ATLAS_COL);
  sc.playpal = SECP(uint8_t, GD_S_PLAYPAL); sc.colormap = SECP(uint8_t, GD_S_COLORMAP);
  sc.sprInfo = SECP(int32_t, GD_S_SPR_INFO); sc.sprAtlas = SECP(uint8_t, GD_S_SPR_ATLAS); sc.sprPost = SECP(uint8_t, GD_S_SPR_POST);
  sc.addLut = SECP(uint8_t, GD_S_ADD_LUT); sc.transLut = SECP(uint8_t, GD_S_TRANS_LUT);
  sc.wpnInfo = SECP(int32_t, GD_S_WPN_INFO); sc.wpnAtlas = SECP(uint8_t, GD_S_WPN_ATLAS); sc.wpnOpaque = SECP(uint8_t, GD_S_WPN_OPAQUE);
  sc.wpnFrameIds = SECP(int32_t, GD_S_WPN_FRAME_IDS); sc.wpnFlashIds = SECP(int32_t, GD_S_WPN_FLASH_IDS);
  sc.wpnFlashLights = SECP(int32_t, GD_S_WPN_FLASH_LIGHTS);
  sc.hudInfo = SECP(int32_t, GD_S_HUD_INFO); sc.hudAtlas = SECP(uint8_t, GD_S_HUD_ATLAS); sc.hudOpaque = SECP(uint8_t, GD_S_HUD_OPAQUE);
  sc.fineSine = SECP(int32_t, GD_S_FINESINE); sc.fineTan = SECP(int32_t, GD_S_FINETAN);
  sc.rayOffsets = SECP(float, GD_S_RAY_OFFSETS); sc.rayCosCorr = SECP(float, GD_S_RAY_COSCORR);
  sc.secBBox = SECP(float, GD_S_SECTOR_BBOX);
  sc.maskedWalls = SECP(int32_t, GD_S_MASKED_WALLS);
  sc.damageAlpha = SECP(float, GD_S_DAMAGE_ALPHA);
  sc.groupH[1] = SECP(float, GD_S_FLOOR_GROUP_H); sc.groupOff[1] = SECP(int32_t, GD_S_FLOOR_GROUP_OFF);
  sc.groupSec[1] = SECP(int32_t, GD_S_FLOOR_GROUP_SEC); sc.groups[1] = h[GD_H_FLOOR_GROUPS];
  sc.groupH[0] = SECP(float, GD_S_CEIL_GROUP_H); sc.groupOff[0] = SECP(int32_t, GD_S_CEIL_GROUP_OFF);
  sc.groupSec[0] = SECP(int32_t, GD_S_CEIL_GROUP_SEC); sc.groups[0] = h[GD_H_CEIL_GROUPS];
  sc.M = h[GD_H_MASKED_WALLS_N];
#undef SECP
  r->smemBytes = gd_shared_bytes(sc.W, max_things);
  r->secWallsN = h[GD_H_SEC_WALLS_N]; r->vtxWallsN = h[GD_H_VTX_WALLS_N]; r->V = h[GD_H_VERTICES];
  r->stageMask = 0;
  int prev = 0;
  if (cudaGetDevice(&prev) != cudaSuccess || cudaSetDevice(device) != cudaSuccess) { delete r; return GD_ERR_CUDA; }
  int maxOptin = 0, sms = 0;
  cudaDeviceGetAttribute(&maxOptin, cudaDevAttrMaxSharedMemoryPerBlockOptin, device);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
  /* stage as many topology tables as the SM's shared memory still holds */
  for (int bit = 1; bit <= GD_STAGE_ROWPROJ; bit <<= 1) {
    size_t extra = gd_stage_bytes(bit, sc.W, sc.S, r->V, r->secWallsN, r->vtxWallsN);
    if (r->smemBytes + extra + 1024 <= (size_t)maxOptin) { r->smemBytes += extra; r->stageMask |= bit; }
  }
  int rc = GD_OK;
  if ((size_t)maxOptin < r->smemBytes) {
    rc = GD_ERR_SHARED;
  } else if (cudaFuncSetAttribute(gd_render_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)r->smemBytes) !=
             cudaSuccess) {
    rc = GD_ERR_CUDA;
  } else {
    int perSm = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&perSm, gd_render_kernel, GD_THREADS, r->smemBytes) != cudaSuccess ||
        perSm < 1)
      rc = GD_ERR_CUDA;
    else
      r->ctas = sms * perSm;  /* one persistent CTA per resident slot */
  }
  r->copyStream = nullptr;
  r->copiesDone = nullptr;
  for (int c = 0; c < GD_HOST_CHUNKS; ++c) r->chunkDone[c] = nullptr;
  if (rc == GD_OK) {
    bool ok = cudaStreamCreateWithFlags(&r->copyStream, cudaStreamNonBlocking) == cudaSuccess &&
              cudaEventCreateWithFlags(&r->copiesDone, cudaEventDisableTiming) == cudaSuccess;
    for (int c = 0; ok && c < GD_HOST_CHUNKS; ++c)
      ok = cudaEventCreateWithFlags(&r->chunkDone[c], cudaEventDisableTiming) == cudaSuccess;
    if (!ok) rc = GD_ERR_CUDA;
  }
  cudaSetDevice(prev);
  if (rc != GD_OK) { cudaGetLastError(); gd_renderer_destroy(r); return rc; }
  *out = r;
  return GD_OK;
}

extern "C" void gd_renderer_destroy(gd_renderer *r) {
  if (!r) return;
  int prev = 0;
  bool switched = cudaGetDevice(&prev) == cudaSuccess && cudaSetDevice(r->device) == cudaSuccess;
  for (int c = 0; c < GD_HOST_CHUNKS; ++c)
    if (r->chunkDone[c]) cudaEventDestroy(r->chunkDone[c]);
  if (r->copiesDone) cudaEventDestroy(r->copiesDone);
  if (r->copyStream) cudaStreamDestroy(r->copyStream);
  if (switched) cudaSetDevice(prev);
  delete r;
}

extern "C" size_t gd_renderer_scratch_bytes(const gd_renderer *r) {
  return r ? (size_t)r->ctas * gd_scratch_per_cta(r->sc.W, r->sc.S) + 16 : 0;
}

extern "C" int gd_renderer_ctas(const gd_renderer *r) { return r ? r->ctas : 0; }
extern "C" size_t gd_renderer_shared_bytes(const gd_renderer *r) { return r ? r->smemBytes : 0; }

static int gd_launch(const gd_renderer *r, const int32_t *lanes, const gd_thing *things, int n, int flags,
                     uint8_t *stack, const uint8_t *reset_mask, uint8_t *obs_out, uint8_t *indexed_out,
                     uint8_t *rgb_out, void *scratch, size_t scratch_bytes, int *status, void *stream) {
  if (!r || !lanes || !scratch || !status) return GD_ERR_NULL;
  if (r->maxThings > 0 && !things) return GD_ERR_NULL;
  if (n < 0) return GD_ERR_SIZE;
  if (n == 0) return GD_OK;
  if (scratch_bytes < gd_renderer_scratch_bytes(r)) return GD_ERR_SCRATCH;
  uintptr_t align = (uintptr_t)lanes | (uintptr_t)things | (uintptr_t)stack | (uintptr_t)obs_out |
                    (uintptr_t)indexed_out | (uintptr_t)rgb_out | (uintptr_t)scratch;
  if (align & 15) return GD_ERR_ALIGN;
  GdParams p;
  p.sc = r->sc;
  p.lanes = lanes; p.things = things; p.maxThings = r->maxThings; p.n = n; p.flags = flags;
  p.stack = stack; p.resetMask = reset_mask; p.obsOut = obs_out; p.indexedOut = indexed_out; p.rgbOut = rgb_out;
  p.scratch = (uint8_t *)scratch; p.status = status;
  p.queueOffset = (size_t)r->ctas * gd_scratch_per_cta(r->sc.W, r->sc.S);
  p.stageMask = r->stageMask; p.secWallsN = r->secWallsN; p.vtxWallsN = r->vtxWallsN; p.V = r->V;
  int grid = n < r->ctas ? n : r->ctas;
  gd_render_kernel<<<grid, GD_THREADS, r->smemBytes, (cudaStream_t)stream>>>(p);
  return cudaGetLastError() == cudaSuccess ? GD_OK : GD_ERR_CUDA;
}

extern "C" int gd_render_step(const gd_renderer *r, const int32_t *lanes, const void *things, int n, int mask_hud,
                              uint8_t *stack, void *scratch, size_t scratch_bytes, int *status, void *stream) {
  if (!stack) return GD_ERR_NULL;
  int flags = GD_F_STACK_ROLL | (mask_hud ? GD_F_MASK_HUD : GD_F_DRAW_HUD);
  return gd_launch(r, lanes, (const gd_thing *)things, n, flags, stack, nullptr, nullptr, nullptr, nullptr, scratch,
                   scratch_bytes, status, stream);
}

extern "C" int gd_render_reset(const gd_renderer *r, const int32_t *lanes, const void *things, int n, int mask_hud,
                               const uint8_t *reset_mask, uint8_t *stack, void *scratch, size_t scratch_bytes,
                               int *status, void *stream) {
  if (!stack || !reset_mask) return GD_ERR_NULL;
  int flags = GD_F_STACK_FILL | (mask_hud ? GD_F_MASK_HUD : GD_F_DRAW_HUD);
  return gd_launch(r, lanes, (const gd_thing *)things, n, flags, stack, reset_mask, nullptr, nullptr, nullptr, scratch,
                   scratch_bytes, status, stream);
}

extern "C" int gd_render_frames(const gd_renderer *r, const int32_t *lanes, const void *things, int n, int mask_hud,
                                int include_hud, uint8_t *obs_out, uint8_t *indexed_out, uint8_t *rgb_out,
                                void *scratch, size_t scratch_bytes, int *status, void *stream) {
  if (!obs_out && !indexed_out && !rgb_out) return GD_ERR_NULL;
  int flags = (mask_hud ? GD_F_MASK_HUD : 0) | ((include_hud || !mask_hud) ? GD_F_DRAW_HUD : 0);
  return gd_launch(r, lanes, (const gd_thing *)things, n, flags, nullptr, nullptr, obs_out, indexed_out, rgb_out,
                   scratch, scratch_bytes, status, stream);
}

extern "C" int gd_render_step_frames(const gd_renderer *r, const int32_t *lanes, const void *things, int n,
                                     int mask_hud, int include_hud, uint8_t *stack, uint8_t *indexed_out,
                                     uint8_t *rgb_out, void *scratch, size_t scratch_bytes, int *status,
                                     void *stream) {
  if (!stack || (!indexed_out && !rgb_out)) return GD_ERR_NULL;
  int flags = GD_F_STACK_ROLL | (mask_hud ? GD_F_MASK_HUD : 0) | ((include_hud || !mask_hud) ? GD_F_DRAW_HUD : 0);
  return gd_launch(r, lanes, (const gd_thing *)things, n, flags, stack, nullptr, nullptr, indexed_out, rgb_out,
                   scratch, scratch_bytes, status, stream);
}

/* Host-buffer variant of gd_render_step: copies the lane and thing records to
 * the caller's device staging buffers, renders, and copies the newest frame of
 * every lane (stack slot 3) back to `obs_host`.  Everything is queued on
 * `stream`; pinned host memory keeps the copies asynchronous. */
extern "C" int gd_render_step_host(const gd_renderer *r, const int32_t *lanes_host, const void *things_host, int n,
                                   int mask_hud, int32_t *lanes_dev, void *things_dev, uint8_t *stack,
                                   uint8_t *obs_host, void *scratch, size_t scratch_bytes, int *status,
                                   void *stream) {
  if (!r || !lanes_host || !lanes_dev || !stack || !obs_host) return GD_ERR_NULL;
  if (r->maxThings > 0 && (!things_host || !things_dev)) return GD_ERR_NULL;
  if (n < 0) return GD_ERR_SIZE;
  if (n == 0) return GD_OK;
  cudaStream_t s = (cudaStream_t)stream;
  size_t thingStride = (size_t)(r->maxThings > 0 ? r->maxThings : 1) * sizeof(gd_thing);
  if (cudaMemcpyAsync(lanes_dev, lanes_host, (size_t)n * GD_LANE_WORDS * 4, cudaMemcpyHostToDevice, s) != cudaSuccess)
    return GD_ERR_CUDA;
  if (things_host &&
      cudaMemcpyAsync(things_dev, things_host, (size_t)n * thingStride, cudaMemcpyHostToDevice, s) != cudaSuccess)
    return GD_ERR_CUDA;
  /* Pinned (or registered) host memory is mapped into the device's address
   * space: the kernel then writes every lane's newest frame straight into it
   * while it draws the following lanes, and no copy is left to wait for. */
  {
    cudaPointerAttributes attr;
    if (cudaPointerGetAttributes(&attr, obs_host) == cudaSuccess && attr.type == cudaMemoryTypeHost &&
        attr.devicePointer != nullptr && (((uintptr_t)attr.devicePointer) & 15) == 0) {
      int flags = GD_F_STACK_ROLL | (mask_hud ? GD_F_MASK_HUD : GD_F_DRAW_HUD);
      return gd_launch(r, lanes_dev, (const gd_thing *)things_dev, n, flags, stack, nullptr,
                       (uint8_t *)attr.devicePointer, nullptr, nullptr, scratch, scratch_bytes, status, stream);
    }
    cudaGetLastError();
  }
  /* Pageable host memory: lanes are drawn in chunks; each chunk's newest frames travel to the host
   * on the side stream while the next chunk is drawn.  The caller's stream
   * waits for the last copy, so synchronising it covers the whole call. */
  const size_t frame = (size_t)GD_OBS * GD_OBS;
  const int chunks = n >= 512 * GD_HOST_CHUNKS ? GD_HOST_CHUNKS : 1;
  const int per = (n + chunks - 1) / chunks;
  for (int c = 0; c < chunks; ++c) {
    const int n0 = c * per, nc = (n0 + per <= n ? per : n - n0);
    if (nc <= 0) break;
    const gd_thing *th = things_dev ? (const gd_thing *)things_dev + (size_t)n0 * (r->maxThings > 0 ? r->maxThings : 1)
                                    : nullptr;
    uint8_t *st = stack + (size_t)n0 * GD_STACK * frame;
    int rc = gd_render_step(r, lanes_dev + (size_t)n0 * GD_LANE_WORDS, th, nc, mask_hud, st, scratch, scratch_bytes,
                            status, stream);
    if (rc != GD_OK) return rc;
    cudaStream_t cs = s;
    if (chunks > 1) {
      cs = r->copyStream;
      if (cudaEventRecord(r->chunkDone[c], s) != cudaSuccess || cudaStreamWaitEvent(cs, r->chunkDone[c], 0) != cudaSuccess)
        return GD_ERR_CUDA;
    }
    if (cudaMemcpy2DAsync(obs_host + (size_t)n0 * frame, frame, st + (GD_STACK - 1) * frame, GD_STACK * frame, frame,
                          (size_t)nc, cudaMemcpyDeviceToHost, cs) != cudaSuccess)
      return GD_ERR_CUDA;
  }
  if (chunks > 1) {
    if (cudaEventRecord(r->copiesDone, r->copyStream) != cudaSuccess ||
        cudaStreamWaitEvent(s, r->copiesDone, 0) != cudaSuccess)
      return GD_ERR_CUDA;
  }
  return GD_OK;
}

/* ---- allocation-free entry point ------------------------------------------
 * gd_render_step for hosts that are not allowed to allocate device memory at
 * all -- for instance a plugin loaded into an inference server or a game
 * process whose memory pool is owned and fully budgeted by its embedder, or
 * code that runs after the framework's allocator has been frozen.  Such a
 * caller cannot obtain the scratch buffer the other entry points ask for, so
 * this variant keeps the clip-event scratch in a fixed array inside the
 * library image.  Every GPU that loads the library holds GD_STATIC_SCRATCH_BYTES
 * of it until the process exits.
 */
#define GD_STATIC_MAX_CTAS 32
#define GD_STATIC_MAX_WALLS 256
/* a scene of W walls has fewer than W sectors (three walls bound a sector, a wall bounds two) */
#define GD_STATIC_PER_CTA ((GD_SCRATCH_FIXED + GD_STATIC_MAX_WALLS * 2 * GD_PLANE_ENTRY_BYTES + \
                            GD_STATIC_MAX_WALLS * 4 * sizeof(GdRowProj) + 31) & ~(size_t)15)
#define GD_STATIC_SCRATCH_BYTES (GD_STATIC_MAX_CTAS * GD_STATIC_PER_CTA + 16)
#define GD_STATIC_MAX_DEVICES 64

static __device__ __align__(256) unsigned char gd_static_scratch[GD_STATIC_SCRATCH_BYTES];

/* device address of the array above, looked up once per device */
static unsigned char *gd_static_scratch_ptr[GD_STATIC_MAX_DEVICES];

extern "C" size_t gd_static_scratch_bytes(void) { return GD_STATIC_SCRATCH_BYTES; }
extern "C" int gd_static_max_walls(void) { return GD_STATIC_MAX_WALLS; }

extern "C" int gd_render_step_static(const gd_renderer *r, const int32_t *lanes, const void *things, int n,
                                     int mask_hud, uint8_t *stack, int *status, void *stream) {
  if (!r || !lanes || !stack || !status) return GD_ERR_NULL;
  if (r->maxThings > 0 && !things) return GD_ERR_NULL;
  if (n < 0) return GD_ERR_SIZE;
  if (r->sc.W > GD_STATIC_MAX_WALLS || r->sc.S > GD_STATIC_MAX_WALLS) return GD_ERR_STATIC_LIMIT;
  if (r->device < 0 || r->device >= GD_STATIC_MAX_DEVICES) return GD_ERR_STATIC_LIMIT;
  if (n == 0) return GD_OK;
  uintptr_t align = (uintptr_t)lanes | (uintptr_t)things | (uintptr_t)stack;
  if (align & 15) return GD_ERR_ALIGN;
  int current = -1;
  if (cudaGetDevice(&current) != cudaSuccess) return GD_ERR_CUDA;
  if (current != r->device) return GD_ERR_DEVICE;  /* the renderer's device must be the current one */
  unsigned char *scratch = gd_static_scratch_ptr[current];
  if (!scratch) {
    /* In host code the array's name is only a handle: the kernel needs the
     * address the symbol has on this device. */
    void *address = nullptr;
    if (cudaGetSymbolAddress(&address, gd_static_scratch) != cudaSuccess || !address) {
      cudaGetLastError();
      return GD_ERR_CUDA;
    }
    scratch = (unsigned char *)address;
    gd_static_scratch_ptr[current] = scratch;
  }
  GdParams p;
  p.sc = r->sc;
  p.lanes = lanes; p.things = (const gd_thing *)things; p.maxThings = r->maxThings; p.n = n;
  p.flags = GD_F_STACK_ROLL | (mask_hud ? GD_F_MASK_HUD : GD_F_DRAW_HUD);
  p.stack = stack; p.resetMask = nullptr; p.obsOut = nullptr; p.indexedOut = nullptr; p.rgbOut = nullptr;
  p.scratch = scratch; p.status = status;
  /* lane queue: the last 16 bytes of the array; zero when the library is
   * loaded and left at zero by every launch */
  p.queueOffset = (size_t)GD_STATIC_MAX_CTAS * GD_STATIC_PER_CTA;
  p.stageMask = r->stageMask; p.secWallsN = r->secWallsN; p.vtxWallsN = r->vtxWallsN; p.V = r->V;
  int grid = n < r->ctas ? n : r->ctas;
  if (grid > GD_STATIC_MAX_CTAS) grid = GD_STATIC_MAX_CTAS;
  gd_render_kernel<<<grid, GD_THREADS, r->smemBytes, (cudaStream_t)stream>>>(p);
  return cudaGetLastError() == cudaSuccess ? GD_OK : GD_ERR_CUDA;
}
