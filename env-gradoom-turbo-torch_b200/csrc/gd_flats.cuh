/* Point-in-sector tests and the per-pixel flat fallback layer.
 * Part of gd_render.cu (one translation unit); not meant to be included elsewhere. */
#ifndef GD_FLATS_CUH
#define GD_FLATS_CUH

/* ---- point in sector (engine.py:9598-9617) ------------------------------ */
/* Crossing parity of a +x ray over the sector's edges.  The bounding box only
 * skips sectors whose parity is provably even. */
__device__ __forceinline__ bool gd_point_in_sector(const GdScene &sc, int s, float px, float py) {
  s = GD_CHECK_SECTOR(s, sc.S);
  const float4 bb = *reinterpret_cast<const float4 *>(&sc.secBBox[s * 4]);
  if (py >= bb.w || py < bb.z) return false;           /* no edge straddles the ray's row */
  if (px > bb.y + 1.0f) return false;                  /* every crossing lies left of the point */
  if (px < bb.x - 1.0f && sc.secI[s * 4 + 3]) return false;  /* closed loops cross an even number of times */
  int crossings = 0;
#pragma unroll 1
  for (int k = sc.edgeOff[s]; k < sc.edgeOff[s + 1]; ++k) {
    const float4 e = *reinterpret_cast<const float4 *>(&sc.walls[GD_CHECK_INDEX(sc.edgeWalls[k], sc.W) * 4]);
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
__device__ __noinline__ bool gd_pixel_unresolved(const GdScene &sc_, const GdView &v_, int x, int y, float rc, float rs,
                                                 int hint) {
  const GdScene &sc = *gd_as_shared(&sc_);
  const GdView &v = *gd_as_shared(&v_);
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

__device__ float gd_plane_depth(const GdScene &sc_, const GdView &v_, int sector, bool isFloor, int y) {
  const GdScene &sc = *gd_as_shared(&sc_);
  const GdView &v = *gd_as_shared(&v_);
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
 * from the nearest anchors left and right; here a pixel that resolves by
 * itself costs one probe, and only when some do not is the repair state built,
 * once per lane and only for the rows that still hold unclaimed pixels. */
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

__device__ __noinline__ GdFlatRay gd_flat_ray(const GdScene &sc_, const GdView &v_, int x) {
  const GdScene &sc = *gd_as_shared(&sc_);
  const GdView &v = *gd_as_shared(&v_);
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

__device__ __noinline__ GdFlatProbe gd_flat_probe(const GdScene &sc_, const GdView &v_, const GdFlatRay &r,
                                                  const GdFlatBounds &b, int y, int currentSector) {
  const GdScene &sc = *gd_as_shared(&sc_);
  const GdView &v = *gd_as_shared(&v_);
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
__device__ void gd_fallback_pass(const GdScene &sc_, const GdView &v_, const GdShared &sh_, int currentSector,
                                 unsigned short *vsec, bool &sweepDone) {
  const GdScene &sc = *gd_as_shared(&sc_);
  const GdView &v = *gd_as_shared(&v_);
  const GdShared &sh = *gd_as_shared(&sh_);
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
      sh.frame[py * GD_SW + px] = (uint8_t)gd_plane_pixel<false>(p, v.center, gd_shared_addr(sh.yslope), gd_shared_addr(sh.colormap), py);
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
    sh.frame[py * GD_SW + px] = (uint8_t)gd_plane_pixel<false>(p, v.center, gd_shared_addr(sh.yslope), gd_shared_addr(sh.colormap), py);
    atomicOr(&owned[(py >> 5) * GD_SW + px], 1u << (py & 31));
  }
  __syncthreads();
}

#endif
