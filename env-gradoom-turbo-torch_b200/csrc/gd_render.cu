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
#define GD_HUD_MAX_PATCHES 48
#define GD_WARPS (GD_THREADS / 32)
#define GD_INF CUDART_INF_F

/* render flags */
#define GD_F_MASK_HUD 1     /* observation sees 32 black rows instead of the status bar */
#define GD_F_DRAW_HUD 2     /* composite the status bar (needed for RGB / unmasked obs) */
#define GD_F_STACK_ROLL 4   /* shift the stack by one slot and append */
#define GD_F_STACK_FILL 8   /* write all four slots of lanes whose mask byte is set */
#define GD_F_WRITE_OBS 16   /* write plain (n,84,84) observations to obsOut */
#define GD_F_STACK_RING 32  /* the stack is a mirrored ring of eight slots per lane (see gd_render_step_ring) */

struct GdParams {
  GdScene sc;
  const int32_t *lanes;
  const gd_thing *things;
  int maxThings;
  int n;
  int flags;
  uint8_t *stack;            /* n x 4 x 84 x 84, or n x 8 x 84 x 84 with GD_F_STACK_RING */
  int ringHead;              /* GD_F_STACK_RING: slot 0..3 that takes the new frame (and slot + 4) */
  const uint8_t *resetMask;  /* n, for GD_F_STACK_FILL */
  uint8_t *obsOut;           /* n x 84 x 84, optional */
  uint8_t *indexedOut;       /* n x 240 x 320, optional */
  uint8_t *rgbOut;           /* n x 240 x 320 x 3, optional */
  uint8_t *scratch;          /* ctas x gd_scratch_per_cta(W), then the lane queue (2 words, zero between launches) */
  size_t queueOffset;
  int stageMask;             /* which scene tables each CTA copies into shared memory */
  int frameRows;             /* rows of the frame kept in shared memory: GD_VIEW_H when neither the status bar
                                nor a full frame is wanted (the 32 rows make room for more tables), else GD_SCREEN_H */
  int secWallsN, vtxWallsN, V;
  int *status;
  const gd_decal *decals;    /* n x decalSlots rings of bullet chips, or null */
  int decalSlots;
  uint8_t *decalScratch;     /* ctas x gd_decal_scratch_per_cta(decalSlots) */
  GdWall *fragScratch;       /* ctas x F fragment records, when the scene has split lines */
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
  unsigned *ownerMask;  /* 10 words: boundary_has_projected_owner; words 16..25: columns whose walk goes on after leaving the map */
  GdWall *walls;        /* W */
  GdWall *frags;        /* scratch: F projection fragments of split lines (only their spans, depths and light) */
  GdActor *actors;      /* maxThings */
  unsigned long long *pal64;  /* 256: R | G<<20 | B<<40 */
  uint8_t *obs;         /* 84 x 84; shares the memory of hitD, which is free once the sprites are drawn */
  int *misc;            /* 16 ints: start sector, fallback queue length, its unresolved rows' range, GdFlatBounds */
  unsigned *masks;      /* 14 x 320: per-column filled / plane-owned row bitmasks */
  unsigned *pal32;      /* 256: the lane's palette as r | g << 8 | b << 16, for the RGB24 output */
  float *maskedDist;    /* 320: nearest masked drawseg of the column ... */
  unsigned *maskedInfo; /* ... its wall << 16 | ceiling clip << 8 | floor clip; 0xFFFF0000 | .. = none */
  float *hitD, *hitA;   /* 8 x 320 each: per-column cache of this iteration's wall hits */
  uint8_t *hitF;        /* 8 x 320 */
};

__host__ __device__ inline size_t gd_align16(size_t v) { return (v + 15) & ~(size_t)15; }

__host__ __device__ inline size_t gd_shared_bytes(int W, int maxThings, int frameRows) {
  size_t b = 0;
  b += gd_align16((size_t)frameRows * GD_SW);
  b += gd_align16(32 * 256);
  b += gd_align16(768);
  b += gd_align16(GD_VH * 4);
  b += gd_align16(GD_LANE_WORDS * 4);
  b += gd_align16(GD_SW * 4);
  b += gd_align16(GD_SW * 2);
  b += gd_align16(32 * 4);
  b += gd_align16(256 * 8);
  b += gd_align16(64);
  b += gd_align16(14 * GD_SW * 4);
  b += 2 * gd_align16(GD_SW * 4);
  b += gd_align16(256 * 4);
  b += 2 * gd_align16(8 * GD_SW * 4) + gd_align16(8 * GD_SW);
  b += gd_align16((size_t)W * sizeof(GdWall));
  b += gd_align16((size_t)(maxThings > 0 ? maxThings : 1) * sizeof(GdActor));
  return b;
}

__device__ inline void gd_carve(uint8_t *base, int W, int maxThings, int frameRows, GdShared &s) {
  size_t o = 0;
  s.frame = base + o; o += gd_align16((size_t)frameRows * GD_SW);
  s.colormap = base + o; o += gd_align16(32 * 256);
  s.playpal = base + o; o += gd_align16(768);
  s.yslope = (unsigned *)(base + o); o += gd_align16(GD_VH * 4);
  s.lane = (int32_t *)(base + o); o += gd_align16(GD_LANE_WORDS * 4);
  s.wallDistance = (float *)(base + o); o += gd_align16(GD_SW * 4);
  s.blockingWall = (short *)(base + o); o += gd_align16(GD_SW * 2);
  s.ownerMask = (unsigned *)(base + o); o += gd_align16(32 * 4);
  s.pal64 = (unsigned long long *)(base + o); o += gd_align16(256 * 8);
  s.misc = (int *)(base + o); o += gd_align16(64);
  s.masks = (unsigned *)(base + o); o += gd_align16(14 * GD_SW * 4);
  s.maskedDist = (float *)(base + o); o += gd_align16(GD_SW * 4);
  s.maskedInfo = (unsigned *)(base + o); o += gd_align16(GD_SW * 4);
  s.pal32 = (unsigned *)(base + o); o += gd_align16(256 * 4);
  s.hitD = (float *)(base + o); o += gd_align16(8 * GD_SW * 4);
  s.hitA = (float *)(base + o); o += gd_align16(8 * GD_SW * 4);
  s.hitF = base + o; o += gd_align16(8 * GD_SW);
  s.obs = (uint8_t *)s.hitD;
  static_assert(8 * GD_SW * 4 >= GD_OBS * GD_OBS && 8 * GD_SW * 4 >= (GD_HUD_MAX_PATCHES + 1) * 16, "obs aliases hitD");
  s.walls = (GdWall *)(base + o); o += gd_align16((size_t)W * sizeof(GdWall));
  s.actors = (GdActor *)(base + o);
}

#include "gd_geometry.cuh"
#include "gd_walk.cuh"
#include "gd_flats.cuh"
#include "gd_sprites.cuh"
#include "gd_decals.cuh"
#include "gd_output.cuh"

/* ---- the kernel ----------------------------------------------------------- */

/* Two instantiations: kSplit = the scene carries projection fragments of split lines. */
template <bool kSplit>
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
    gd_carve(gd_smem, sc.W, p.maxThings, p.frameRows, sh);
    uint8_t *cursor = gd_smem + gd_shared_bytes(sc.W, p.maxThings, p.frameRows);
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
    sh.frags = p.fragScratch ? p.fragScratch + (size_t)blockIdx.x * sc.F : nullptr;
    if (!sh.frags) sc.F = 0;
    if (tid == 0) { sScene = sc; sShared = sh; }
  }
  __syncthreads();
  const GdScene &sc = sScene;
  const GdShared &sh = sShared;
#ifdef GD_CHECKED
  if (tid == 0) gdCheckedStatus = p.status;
  __syncthreads();
#endif
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
    if (p.flags & GD_F_STACK_FILL) {
      if (p.resetMask && !p.resetMask[l]) continue;  /* uniform across the CTA */
    }
    if (tid < GD_LANE_WORDS) sh.lane[tid] = p.lanes[(size_t)l * GD_LANE_WORDS + tid];
    if (tid < 10) { sh.ownerMask[tid] = 0; sh.ownerMask[16 + tid] = 0; }
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
#ifdef GD_CHECKED
    {
      /* a lane whose pose is not a number, or lies far outside any map, is drawn from the map's origin instead */
      const float lx = __int_as_float(sh.lane[GD_L_X]), ly = __int_as_float(sh.lane[GD_L_Y]);
      const float lz = __int_as_float(sh.lane[GD_L_VIEW_Z]), la = __int_as_float(sh.lane[GD_L_ANGLE]);
      const bool badPose = !isfinite(lx) || !isfinite(ly) || !isfinite(lz) || !isfinite(la) || fabsf(lx) > 32768.0f ||
                           fabsf(ly) > 32768.0f;
      const int weapon = sh.lane[GD_L_WEAPON];
      __syncthreads();
      if (tid == 0) {
        GD_FLAG_STATE(badPose || weapon < 0 || weapon > 7 || sh.lane[GD_L_THINGS] < 0);
        if (badPose) {
          sh.lane[GD_L_X] = sh.lane[GD_L_Y] = sh.lane[GD_L_ANGLE] = 0;
          sh.lane[GD_L_X_FIXED] = sh.lane[GD_L_Y_FIXED] = sh.lane[GD_L_ANGLE_BAM] = 0;
          sh.lane[GD_L_VIEW_Z] = __float_as_int(41.0f);
        }
      }
      __syncthreads();
    }
#endif
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
    if (kSplit)
      for (int f = tid; f < sc.F; f += GD_THREADS) gd_project_fragment(sc, v, f, sh.frags[f]);
    for (int idx = GD_THREADS - 1 - tid; idx < sc.S * 2; idx += GD_THREADS)   /* the threads the walls leave idle */
      gd_plane_entry_setup(sc, v, idx >> 1, (idx & 1) != 0, sh.planeTab[idx]);
    for (int a = tid; a < nThings; a += GD_THREADS) {
      int sector = pointSector[a] == 0x7fffffff ? 0 : pointSector[a];
      gd_actor_setup(sc, v, p.things[(size_t)l * p.maxThings + a], sector, sh.actors[a]);
    }
    if (tid == GD_THREADS - 1) sh.misc[0] = pointSector[64] == 0x7fffffff ? 0 : pointSector[64];
    __syncthreads();
    gd_wall_spans(sc, v, sh);
    /* row projection tables, for the walls that passed the frustum test (the
     * walk selects no other wall) */
    for (int idx = tid; idx < sh.misc[2] * 4; idx += GD_THREADS) {
      int w = ((const short *)sh.hitD)[idx >> 2], slot = idx & 3;
      int sector = gd_wsec(sc, w * 2 + (slot >> 1));
      if (sector >= 0) gd_rowproj_setup(v, sh.walls[w], sc.secF[sector * 2 + (slot & 1)], rowproj[w * 4 + slot]);
    }
    __syncthreads();
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
    gd_mark_afterlife_columns(sc, sh);
    {
      float rx, ry, wd;
      int bw;
      gd_ray(v, tid, rx, ry);
      gd_blocking_raycast(sc, v, sh, frustumList, frustumListed, rx, ry, wd, bw);
      sh.wallDistance[tid] = wd;
      sh.blockingWall[tid] = (short)bw;
    }
    __syncthreads();
    gd_walk<kSplit>(sc, v, sh, events, eventCount, rowproj, p.status, sh.misc[0]);
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
      gd_masked_pass<kSplit>(sc, v, sh);
      __syncthreads();
    }
#ifndef GD_NO_DECALS
    if (p.decals != nullptr && sc.decals > 0)
      gd_decals(sc, v, sh, events, eventCount, p.decals + (size_t)l * p.decalSlots, p.decalSlots,
                p.decalScratch + (size_t)blockIdx.x * gd_decal_scratch_per_cta(p.decalSlots));
#endif
    gd_sprites(sc, v, sh, events, eventCount, nThings);
    __syncthreads();
    gd_weapon(sc, sh.lane, sh.frame);
    __syncthreads();
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
      if (p.stack && (p.flags & GD_F_STACK_RING)) {
        /* mirrored ring: no old slot is read or moved */
        uint4 *s0 = (uint4 *)(p.stack + (size_t)l * 2 * GD_STACK * GD_OBS * GD_OBS);
        if (p.flags & GD_F_STACK_FILL) {
          for (int i = tid; i < vecs; i += GD_THREADS) {
            uint4 val = src[i];
#pragma unroll
            for (int k = 0; k < 2 * GD_STACK; ++k) s0[k * vecs + i] = val;
          }
        } else {
          for (int i = tid; i < vecs; i += GD_THREADS) {
            uint4 val = src[i];
            s0[p.ringHead * vecs + i] = val;
            s0[(p.ringHead + GD_STACK) * vecs + i] = val;
          }
        }
      } else if (p.stack) {
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
  if (tid == 0) {
    __threadfence();
    if (atomicAdd(&queue[1], 1u) == gridDim.x - 1) {
      queue[0] = 0;
      queue[1] = 0;
      __threadfence();
    }
  }
}

#include "gd_abi.cuh"
#include "gd_state.cuh"
#include "gd_state_abi.cuh"
#include "gd_move.cuh"
