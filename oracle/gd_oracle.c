/*
 * CPU restatement of the reference's native render-to-observation path.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker for the CUDA library: it
 * is built and called by the tests, by the smoke check and by the CPU-baseline
 * leg of the benchmark, and never by the product path.
 *
 * It restates, as scalar per-lane / per-column C, what the reference computes
 * with batched tensor ops in src/gradoom/engine.py:
 *   wall projection            10747-10869  (project_wall)
 *   wallscan light             11207-11302  (wall_visibility)
 *   PrepWall texture mapping   10672-10739  (prep_wall)
 *   ray / span ownership       11304-11460  (lane_intersections)
 *   blocking ray cast          10534-10557  (blocking_raycast)
 *   per-column portal walk     11462-13371  (wall_pass)
 *   row bounds (OWallMost)     12294-12605  (project_rows)
 *   visplane fill              13372-13422, 10879-10954, 10588-10616 (plane_pass)
 *   sprites                    14138-14228, 14684-14947 (sprite_pass)
 *   thing resolution           14011-14104, 14328-14682 (gd_oracle_resolve_things)
 *   weapon                     14949-15121  (weapon_pass)
 *   status bar                 15158-15267  (hud_pass)
 *   palette + area resize      15381-15434 and the integer twin
 *                              src/gradoom/_triton_kernels.py:120-177
 *   frame stack                9545-9548, 2443-2450
 * Pinned against fixtures produced by running the reference itself
 * (tests/golden/make_golden.py); see tests/test_oracle_golden.py.
 *
 * Float32 expressions keep the reference's operation order; compile with
 * -ffp-contract=off so no multiply-add is fused.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#include "../include/gradoom_b200_layout.h"

#define FU 65536LL
#define SW GD_SCREEN_W
#define VH GD_VIEW_H
#define ANG90 (1LL << 30)
#define FOCAL_X (160LL * FU)
#define Y_ASPECT ((320LL * FU * 240LL) / (200LL * 320LL))
#define FOCAL_Y (160LL * Y_ASPECT)
#define FLOOR_VIS ((160LL * FU * (8LL * FU)) / FOCAL_Y)
#define WALL_VIS (((FOCAL_Y * (320LL * 600LL) / (320LL * 240LL * 3LL)) * (8LL * FU)) >> 16)
#define SPRITE_MIN_DEPTH (2048LL * 4LL)
#define U32MASK 0xFFFFFFFFLL

typedef int64_t i64;

typedef struct {
  const int32_t *hdr;
  const uint8_t *base;
  int W, S, T, texH, texW, P, sprH, sprW, Q, wpnH, wpnW, wpnTics, nStarts, deathF, xdeathF, B;
  int nbDirect, wpnAvailable;
  const float *walls;
  const int32_t *wsec;
  const float *wlen;
  const int32_t *sideTex;
  const float *sideOff;
  const int32_t *wvtx, *vtxOff, *vtxWalls;
  const int32_t *nbDirectTab, *nbOff, *nbIdx, *nbFlags;
  const int32_t *sbStartOff, *sbStartIdx, *sbEndOff, *sbEndIdx;
  const float *secF;
  const int32_t *secI;
  const int32_t *secOff, *secWalls, *edgeOff, *edgeWalls, *blocking;
  const int32_t *texInfo;
  const float *damageAlpha;
  const uint8_t *texAtlas, *playpal, *colormap;
  const int32_t *sprInfo;
  const uint8_t *sprAtlas, *sprPost;
  const int32_t *enemyWalk, *enemyAttack, *enemyPain, *deathIds, *deathCounts, *deathEnds;
  const int32_t *xdeathIds, *xdeathCounts, *xdeathEnds;
  const int32_t *projFlight, *projExplIds, *projExplCounts, *projExplEnds, *projExplTotal;
  const int32_t *fogIds, *puffIds, *staticIds;
  const uint8_t *addLut, *transLut;
  const int32_t *wpnInfo;
  const uint8_t *wpnAtlas, *wpnOpaque;
  const int32_t *wpnFrameIds, *wpnFlashIds, *wpnFlashLights;
  const int32_t *hudInfo;
  const uint8_t *hudAtlas, *hudOpaque;
  const int32_t *fineSine, *fineTan;
  const float *starts;
  const float *rayOffsets, *rayCosCorr;
  int decals, decalH, decalW;
  int F;                               /* projection fragments of split lines */
  const int32_t *fragOff, *fragFixed;
  const int32_t *decalInfo, *wallFine;
  const uint8_t *decalAtlas, *decalOpacity, *decalBlack;
} Scene;

static const void *sec_ptr(const uint8_t *blob, int s) {
  const int32_t *h = (const int32_t *)blob;
  return blob + h[GD_HDR_SECTION0 + s];
}

static int scene_open(Scene *sc, const uint8_t *blob) {
  const int32_t *h = (const int32_t *)blob;
  if (h[GD_H_MAGIC] != GD_MAGIC || h[GD_H_VERSION] != GD_VERSION) return -1;
  sc->hdr = h;
  sc->base = blob;
  sc->W = h[GD_H_WALLS];
  sc->S = h[GD_H_SECTORS];
  sc->T = h[GD_H_TEXTURES];
  sc->texH = h[GD_H_TEX_H];
  sc->texW = h[GD_H_TEX_W];
  sc->P = h[GD_H_SPRITES];
  sc->sprH = h[GD_H_SPR_H];
  sc->sprW = h[GD_H_SPR_W];
  sc->Q = h[GD_H_WPN_PATCHES];
  sc->wpnH = h[GD_H_WPN_H];
  sc->wpnW = h[GD_H_WPN_W];
  sc->wpnTics = h[GD_H_WPN_TICS];
  sc->nStarts = h[GD_H_STARTS];
  sc->deathF = h[GD_H_DEATH_FRAMES];
  sc->xdeathF = h[GD_H_XDEATH_FRAMES];
  sc->B = h[GD_H_BLOCKING];
  sc->nbDirect = h[GD_H_NB_DIRECT];
  sc->wpnAvailable = h[GD_H_WPN_AVAILABLE];
  sc->walls = sec_ptr(blob, GD_S_WALLS);
  sc->wsec = sec_ptr(blob, GD_S_WALL_SECTORS);
  sc->wlen = sec_ptr(blob, GD_S_WALL_LEN);
  sc->sideTex = sec_ptr(blob, GD_S_SIDE_TEX);
  sc->sideOff = sec_ptr(blob, GD_S_SIDE_OFF);
  sc->wvtx = sec_ptr(blob, GD_S_WALL_VTX);
  sc->vtxOff = sec_ptr(blob, GD_S_VTX_OFF);
  sc->vtxWalls = sec_ptr(blob, GD_S_VTX_WALLS);
  sc->nbDirectTab = sec_ptr(blob, GD_S_NB_DIRECT);
  sc->nbOff = sec_ptr(blob, GD_S_NB_OFF);
  sc->nbIdx = sec_ptr(blob, GD_S_NB_IDX);
  sc->nbFlags = sec_ptr(blob, GD_S_NB_FLAGS);
  sc->sbStartOff = sec_ptr(blob, GD_S_SB_START_OFF);
  sc->sbStartIdx = sec_ptr(blob, GD_S_SB_START_IDX);
  sc->sbEndOff = sec_ptr(blob, GD_S_SB_END_OFF);
  sc->sbEndIdx = sec_ptr(blob, GD_S_SB_END_IDX);
  sc->secF = sec_ptr(blob, GD_S_SECTOR_F);
  sc->secI = sec_ptr(blob, GD_S_SECTOR_I);
  sc->secOff = sec_ptr(blob, GD_S_SEC_OFF);
  sc->secWalls = sec_ptr(blob, GD_S_SEC_WALLS);
  sc->edgeOff = sec_ptr(blob, GD_S_EDGE_OFF);
  sc->edgeWalls = sec_ptr(blob, GD_S_EDGE_WALLS);
  sc->blocking = sec_ptr(blob, GD_S_BLOCKING);
  sc->texInfo = sec_ptr(blob, GD_S_TEX_INFO);
  sc->damageAlpha = sec_ptr(blob, GD_S_DAMAGE_ALPHA);
  sc->texAtlas = sec_ptr(blob, GD_S_TEX_ATLAS);
  sc->playpal = sec_ptr(blob, GD_S_PLAYPAL);
  sc->colormap = sec_ptr(blob, GD_S_COLORMAP);
  sc->sprInfo = sec_ptr(blob, GD_S_SPR_INFO);
  sc->sprAtlas = sec_ptr(blob, GD_S_SPR_ATLAS);
  sc->sprPost = sec_ptr(blob, GD_S_SPR_POST);
  sc->enemyWalk = sec_ptr(blob, GD_S_ENEMY_WALK);
  sc->enemyAttack = sec_ptr(blob, GD_S_ENEMY_ATTACK);
  sc->enemyPain = sec_ptr(blob, GD_S_ENEMY_PAIN);
  sc->deathIds = sec_ptr(blob, GD_S_DEATH_IDS);
  sc->deathCounts = sec_ptr(blob, GD_S_DEATH_COUNTS);
  sc->deathEnds = sec_ptr(blob, GD_S_DEATH_ENDS);
  sc->xdeathIds = sec_ptr(blob, GD_S_XDEATH_IDS);
  sc->xdeathCounts = sec_ptr(blob, GD_S_XDEATH_COUNTS);
  sc->xdeathEnds = sec_ptr(blob, GD_S_XDEATH_ENDS);
  sc->projFlight = sec_ptr(blob, GD_S_PROJ_FLIGHT);
  sc->projExplIds = sec_ptr(blob, GD_S_PROJ_EXPL_IDS);
  sc->projExplCounts = sec_ptr(blob, GD_S_PROJ_EXPL_COUNTS);
  sc->projExplEnds = sec_ptr(blob, GD_S_PROJ_EXPL_ENDS);
  sc->projExplTotal = sec_ptr(blob, GD_S_PROJ_EXPL_TOTAL);
  sc->fogIds = sec_ptr(blob, GD_S_FOG_IDS);
  sc->puffIds = sec_ptr(blob, GD_S_PUFF_IDS);
  sc->staticIds = sec_ptr(blob, GD_S_STATIC_IDS);
  sc->addLut = sec_ptr(blob, GD_S_ADD_LUT);
  sc->transLut = sec_ptr(blob, GD_S_TRANS_LUT);
  sc->wpnInfo = sec_ptr(blob, GD_S_WPN_INFO);
  sc->wpnAtlas = sec_ptr(blob, GD_S_WPN_ATLAS);
  sc->wpnOpaque = sec_ptr(blob, GD_S_WPN_OPAQUE);
  sc->wpnFrameIds = sec_ptr(blob, GD_S_WPN_FRAME_IDS);
  sc->wpnFlashIds = sec_ptr(blob, GD_S_WPN_FLASH_IDS);
  sc->wpnFlashLights = sec_ptr(blob, GD_S_WPN_FLASH_LIGHTS);
  sc->hudInfo = sec_ptr(blob, GD_S_HUD_INFO);
  sc->hudAtlas = sec_ptr(blob, GD_S_HUD_ATLAS);
  sc->hudOpaque = sec_ptr(blob, GD_S_HUD_OPAQUE);
  sc->fineSine = sec_ptr(blob, GD_S_FINESINE);
  sc->fineTan = sec_ptr(blob, GD_S_FINETAN);
  sc->starts = sec_ptr(blob, GD_S_STARTS);
  sc->rayOffsets = sec_ptr(blob, GD_S_RAY_OFFSETS);
  sc->rayCosCorr = sec_ptr(blob, GD_S_RAY_COSCORR);
  sc->decals = h[GD_H_DECALS];
  sc->decalH = h[GD_H_DECAL_H];
  sc->decalW = h[GD_H_DECAL_W];
  sc->decalInfo = sec_ptr(blob, GD_S_DECAL_INFO);
  sc->decalAtlas = sec_ptr(blob, GD_S_DECAL_ATLAS);
  sc->decalOpacity = sec_ptr(blob, GD_S_DECAL_OPACITY);
  sc->decalBlack = sec_ptr(blob, GD_S_DECAL_BLACK);
  sc->wallFine = sec_ptr(blob, GD_S_WALL_FINE);
  sc->F = h[GD_H_FRAGMENTS];
  sc->fragOff = sec_ptr(blob, GD_S_FRAG_OFF);
  sc->fragFixed = sec_ptr(blob, GD_S_FRAG_FIXED);
  return 0;
}

/* ---- small helpers ------------------------------------------------------ */

static inline i64 imin(i64 a, i64 b) { return a < b ? a : b; }
static inline i64 imax(i64 a, i64 b) { return a > b ? a : b; }
static inline i64 iclamp(i64 v, i64 lo, i64 hi) { return v < lo ? lo : (v > hi ? hi : v); }
static inline i64 wrap_mul(i64 a, i64 b) { return (i64)((uint64_t)a * (uint64_t)b); }
static inline i64 shl(i64 a, int k) { return (i64)((uint64_t)a << k); }
/* round-half-to-even of a float32 value to int64 (torch.round + .to(int64)) */
static inline i64 rint_f(float v) { return (i64)rintf(v); }
static inline i64 pymod(i64 a, i64 m) { i64 r = a % m; return (r != 0 && ((r < 0) != (m < 0))) ? r + m : r; }

typedef struct {
  /* view */
  float x, y, angle, viewZ;
  i64 vx, vy, bam, pitchBam;
  i64 vsin, vcos;
  float fcos, fsin;
  i64 center; /* center_fixed */
  int flashLight;
} View;

typedef struct {
  /* FWallCoords, view-ordered endpoints */
  i64 sl, sr, dl, dr;
  /* stored endpoint order view coordinates */
  i64 tx[2], ty[2];
  /* wallscan light per side: left value, step, screen_left */
  i64 visL[2], visStep[2], visSl[2];
  /* span ownership of the ray test */
  i64 isl, isr;
  int hasColumns;
  int frontFacingF; /* float test */
  int oneSided;
} WallView;

typedef struct {
  int W;
  WallView *wv;
  WallView *frag;  /* [F] FWallCoords and wallscan light of every projection fragment */
  float *dist;     /* [SW][W] inf when invalid */
  float *along;    /* clamped to [0,1] */
  uint8_t *geo, *proj, *left;
  int32_t *eoIdx;  /* endpoint owner index */
  float *eoDist;
  uint8_t boundaryHasProjectedOwner[SW];
  float dirx[SW], diry[SW];
  float wallDistance[SW];
  int blockingWall[SW];
} LaneGeom;

static void view_setup(const Scene *sc, const int32_t *lane, View *v) {
  const float *lf = (const float *)lane;
  v->x = lf[GD_L_X];
  v->y = lf[GD_L_Y];
  v->angle = lf[GD_L_ANGLE];
  v->viewZ = lf[GD_L_VIEW_Z];
  v->vx = lane[GD_L_X_FIXED];
  v->vy = lane[GD_L_Y_FIXED];
  v->bam = (i64)(uint32_t)lane[GD_L_ANGLE_BAM];
  v->pitchBam = lane[GD_L_PITCH_BAM];
  i64 fine = (v->bam >> 19) & 8191;
  v->vsin = sc->fineSine[fine];
  v->vcos = sc->fineSine[(fine + 2048) & 8191];
  v->fsin = (float)v->vsin / 65536.0f;
  v->fcos = (float)v->vcos / 65536.0f;
  i64 ti = iclamp((ANG90 - v->pitchBam) >> 19, 0, 4095);
  v->center = 104 * FU + ((FOCAL_Y * (i64)sc->fineTan[ti]) >> 16);
  /* weapon flash light (engine.py:14949-14967) */
  int weapon = (int)iclamp(lane[GD_L_WEAPON], 0, 7);
  int cooldown = (int)iclamp(lane[GD_L_WPN_COOLDOWN], 0, sc->wpnTics - 1);
  int parity = (int)pymod(lane[GD_L_WPN_FIRE_COUNT], 2);
  if (weapon == 1 && cooldown == 0) parity = (int)pymod(imax(lane[GD_L_WPN_READY_TICS] - 1, 0) / 4, 2);
  v->flashLight = sc->wpnFlashLights[(weapon * 2 + parity) * sc->wpnTics + cooldown];
}

static i64 wall_fixed(const Scene *sc, int w, int k) { return rint_f(sc->walls[w * 4 + k] * 65536.0f); }

/* FWallCoords for one ordered endpoint pair (engine.py:10791-10869). */
static void fwall_coords(i64 tx1, i64 ty1, i64 tx2, i64 ty2, i64 *sl, i64 *sr, i64 *dl, i64 *dr) {
  i64 cf = 160 * FU;
  i64 sty1 = ty1 == 0 ? 1 : ty1, sty2 = ty2 == 0 ? 1 : ty2;
  i64 lp = (cf + (tx1 * cf) / sty1) >> 16;
  lp += (tx1 >= 0);
  if (tx1 >= 0) lp = imin(lp, SW);
  i64 rp = (cf + (tx2 * cf) / sty2) >> 16;
  rp += (tx2 >= 0);
  if (tx2 >= 0) rp = imin(rp, SW);
  i64 lden = tx1 - tx2 - ty2 + ty1, rden = ty2 - ty1 - tx2 + tx1;
  i64 slden = lden == 0 ? 1 : lden, srden = rden == 0 ? 1 : rden;
  int lin = tx1 >= -ty1, rin = tx2 <= ty2;
  i64 screenL = lin ? lp : 0, screenR = rin ? rp : SW;
  i64 depthL = lin ? ty1 : ty1 + ((ty2 - ty1) * (tx1 + ty1)) / slden;
  i64 depthR = rin ? ty2 : ty1 + ((ty2 - ty1) * (tx1 - ty1)) / srden;
  int invL = (lin ? ((tx1 > ty1) || (ty1 == 0)) : ((tx2 < -ty2) || (lden == 0))) || (depthL < 32);
  int invR = (rin ? ((tx2 < -ty2) || (ty2 == 0)) : ((tx1 > ty1) || (rden == 0))) || (depthR < 32);
  int inv = invL || invR || (screenR <= screenL);
  if (inv) screenR = screenL;
  *sl = screenL; *sr = screenR; *dl = depthL; *dr = depthR;
}

/* wallscan light interpolation for one endpoint order (engine.py:11217-11291) */
static void wall_visibility(i64 tx1, i64 ty1, i64 tx2, i64 ty2, i64 *visL, i64 *visStep, i64 *visSl) {
  i64 cf = 160 * FU;
  i64 sty1 = ty1 == 0 ? 1 : ty1, sty2 = ty2 == 0 ? 1 : ty2;
  i64 lp = ((cf + (tx1 * cf) / sty1) >> 16) + (tx1 >= 0);
  i64 rp = ((cf + (tx2 * cf) / sty2) >> 16) + (tx2 >= 0);
  i64 lden = tx1 - tx2 - ty2 + ty1, rden = ty2 - ty1 - tx2 + tx1;
  i64 slden = lden == 0 ? 1 : lden, srden = rden == 0 ? 1 : rden;
  int lin = tx1 >= -ty1, rin = tx2 <= ty2;
  i64 wsl = lin ? lp : 0, wsr = rin ? rp : SW;
  i64 wdl = lin ? ty1 : ty1 + ((ty2 - ty1) * (tx1 + ty1)) / slden;
  i64 wdr = rin ? ty2 : ty1 + ((ty2 - ty1) * (tx1 - ty1)) / srden;
  i64 ll = (WALL_VIS << 12) / imax(wdl, 1);
  i64 lr = (WALL_VIS << 12) / imax(wdr, 1);
  *visStep = (lr - ll) / imax(wsr - wsl, 1);
  *visL = ll;
  *visSl = wsl;
}

/* View coordinates, FWallCoords and wallscan light of a segment given by its 16.16 endpoints. */
static void project_fixed(const View *v, const i64 fx[2], const i64 fy[2], WallView *wv) {
  for (int e = 0; e < 2; ++e) {
    i64 rx = fx[e] - v->vx, ry = fy[e] - v->vy;
    wv->tx[e] = (rx * v->vsin - ry * v->vcos) >> 20;
    wv->ty[e] = (rx * v->vcos + ry * v->vsin) >> 20;
  }
  i64 wvx = fx[1] - fx[0], wvy = fy[1] - fy[0];
  i64 fsx = v->vx - fx[0], fsy = v->vy - fy[0];
  int ff = (wvx * fsy - wvy * fsx) < 0;
  int a = ff ? 0 : 1, b = ff ? 1 : 0;
  fwall_coords(wv->tx[a], wv->ty[a], wv->tx[b], wv->ty[b], &wv->sl, &wv->sr, &wv->dl, &wv->dr);
  wall_visibility(wv->tx[0], wv->ty[0], wv->tx[1], wv->ty[1], &wv->visL[0], &wv->visStep[0], &wv->visSl[0]);
  wall_visibility(wv->tx[1], wv->ty[1], wv->tx[0], wv->ty[0], &wv->visL[1], &wv->visStep[1], &wv->visSl[1]);
}

static void lane_geometry(const Scene *sc, const View *v, LaneGeom *g) {
  int W = sc->W;
  g->W = W;
  for (int x = 0; x < SW; ++x) {
    float c = ((float)x - 160.0f) / 160.0f;
    g->dirx[x] = v->fcos + v->fsin * c;
    g->diry[x] = v->fsin - v->fcos * c;
  }
  /* the pieces of the lines a node builder split: the same projection, from their own
   * fixed-point endpoints (engine.py:11478-11500, 10747-10869) */
  for (int f = 0; f < sc->F; ++f) {
    const int32_t *q = &sc->fragFixed[f * 4];
    i64 fx[2] = {q[0], q[2]}, fy[2] = {q[1], q[3]};
    project_fixed(v, fx, fy, &g->frag[f]);
  }
  for (int w = 0; w < W; ++w) {
    WallView *wv = &g->wv[w];
    i64 fx[2] = {wall_fixed(sc, w, 0), wall_fixed(sc, w, 2)};
    i64 fy[2] = {wall_fixed(sc, w, 1), wall_fixed(sc, w, 3)};
    project_fixed(v, fx, fy, wv);
    wv->oneSided = sc->wsec[w * 2 + 1] < 0;

    /* float ray tests for every column (engine.py:11317-11331) */
    const float *wl = &sc->walls[w * 4];
    float sx = wl[0], sy = wl[1];
    float segx = wl[2] - sx, segy = wl[3] - sy;
    float offx = sx - v->x, offy = sy - v->y;
    int first = -1, last = -1;
    for (int x = 0; x < SW; ++x) {
      float rx = g->dirx[x], ry = g->diry[x];
      float den = rx * segy - ry * segx;
      int small = fabsf(den) < 1e-6f;
      float safe = small ? 1.0f : den;
      float distance = (offx * segy - offy * segx) / safe;
      float al = (offx * ry - offy * rx) / safe;
      int geo = !small && distance > 0 && al >= 0 && al <= 1;
      g->geo[x * W + w] = (uint8_t)geo;
      g->dist[x * W + w] = distance;  /* validity applied below */
      g->proj[x * W + w] = (uint8_t)(!small && distance > 0);
      float ac = al;
      if (!(ac >= 0.0f)) ac = ac != ac ? ac : 0.0f;
      if (ac > 1.0f) ac = 1.0f;
      g->along[x * W + w] = ac;
      if (geo) { if (first < 0) first = x; last = x; }
    }
    int hasColumns = first >= 0;
    i64 isl = hasColumns ? first : 0;
    i64 isr = hasColumns ? last + 1 : SW; /* argmax of all-false is 0: last = 319 */
    /* endpoint overrides (engine.py:11359-11427) */
    i64 cf = 160 * FU;
    i64 ecol[2];
    int evis[2];
    for (int e = 0; e < 2; ++e) {
      i64 ty = wv->ty[e], tx = wv->tx[e];
      i64 sty = ty == 0 ? 1 : ty;
      i64 pf = cf + (tx * cf) / sty;
      ecol[e] = (pf >> 16) + (tx >= 0);
      evis[e] = ty > 0 && tx >= -ty && tx <= ty && ecol[e] >= 0 && ecol[e] <= SW;
    }
    float vfsx = v->x - sx, vfsy = v->y - sy; /* origin - start */
    int fff = (segx * vfsy - segy * vfsx) < 0;
    wv->frontFacingF = fff;
    for (int e = 0; e < 2; ++e) {
      int visible = evis[e] && hasColumns;
      int ownsLeft = fff ? (e == 0) : (e == 1);
      if (visible && ownsLeft) isl = ecol[e];
      if (visible && !ownsLeft) isr = ecol[e];
    }
    int oa = fff ? 0 : 1, ob = fff ? 1 : 0;
    int exact = evis[0] && evis[1];
    if (exact) {
      isl = ecol[oa];
      isr = ecol[ob];
      hasColumns = isr > isl;
    }
    hasColumns = hasColumns && (wv->sr > wv->sl);
    wv->isl = isl; wv->isr = isr; wv->hasColumns = hasColumns;
    for (int x = 0; x < SW; ++x) {
      int screenValid = hasColumns && x >= isl && x < isr;
      int pv = g->proj[x * W + w] && screenValid;
      g->proj[x * W + w] = (uint8_t)pv;
      int valid = wv->oneSided ? (pv && fff) : (g->geo[x * W + w] || pv);
      if (!valid) g->dist[x * W + w] = INFINITY;
      g->left[x * W + w] = (uint8_t)(x == isl);
    }
  }
  /* boundary_has_projected_owner and endpoint owners (engine.py:11589-11734) */
  for (int x = 0; x < SW; ++x) {
    const float *D = &g->dist[x * W];
    const uint8_t *PJ = &g->proj[x * W], *LE = &g->left[x * W];
    int any = 0;
    for (int w = 0; w < W; ++w) any |= (LE[w] && isfinite(D[w]));
    g->boundaryHasProjectedOwner[x] = (uint8_t)any;
    for (int w = 0; w < W; ++w) {
      const WallView *wv = &g->wv[w];
      float d = D[w];
      float tol = fmaxf(fabsf(d) / 128.0f, 4.0f);
      int subpixel = (wv->sr - wv->sl <= 1) && !wv->oneSided;
      int usesStart = g->along[x * W + w] <= 0.5f;
      int ownerIdx = w;
      float ownerDist = d;
      int ownerValid = 0;
      if (sc->nbDirect) {
        const int32_t *nd = &sc->nbDirectTab[w * 4];
        int sIdx = nd[0] >= 0 ? nd[0] : w, eIdx = nd[1] >= 0 ? nd[1] : w;
        int hasS = nd[0] >= 0, hasE = nd[1] >= 0;
        int rIdx = usesStart ? sIdx : eIdx, rSlot = usesStart ? nd[2] : nd[3], rHas = usesStart ? hasS : hasE;
        int oIdx = usesStart ? eIdx : sIdx, oSlot = usesStart ? nd[3] : nd[2], oHas = usesStart ? hasE : hasS;
        float rDist = D[rIdx], oDist = D[oIdx];
        int rOwns = rHas && PJ[rIdx] && LE[rIdx];
        int oOwns = subpixel && oHas && PJ[oIdx] && LE[oIdx] && (fabsf(oDist - d) <= tol);
        int useO = oOwns && (!rOwns || oDist < rDist || (oDist == rDist && oSlot < rSlot));
        ownerIdx = useO ? oIdx : rIdx;
        ownerDist = useO ? oDist : rDist;
        ownerValid = rOwns || oOwns;
      } else {
        float best = INFINITY;
        int bestSlot = 0;
        int n0 = sc->nbOff[w], n1 = sc->nbOff[w + 1];
        for (int k = n0; k < n1; ++k) {
          int nb = sc->nbIdx[k], fl = sc->nbFlags[k];
          int rayNb = usesStart ? (fl & 1) : ((fl >> 1) & 1);
          int sel = rayNb || (subpixel && (fabsf(D[nb] - d) <= tol));
          float cand = (PJ[nb] && LE[nb] && sel) ? D[nb] : INFINITY;
          if (cand < best) { best = cand; bestSlot = k - n0; }
        }
        ownerDist = best;
        ownerIdx = (n1 > n0) ? sc->nbIdx[n0 + bestSlot] : w;
        ownerValid = isfinite(best);
      }
      int has = !PJ[w] && ownerValid;
      g->eoIdx[x * W + w] = has ? ownerIdx : w;
      g->eoDist[x * W + w] = has ? ownerDist : d;
    }
  }
  /* blocking ray cast (engine.py:10534-10557) */
  for (int x = 0; x < SW; ++x) {
    float best = INFINITY;
    int bestSlot = 0;
    float rx = g->dirx[x], ry = g->diry[x];
    for (int b = 0; b < sc->B; ++b) {
      const float *wl = &sc->walls[sc->blocking[b] * 4];
      float sx = wl[0], sy = wl[1];
      float segx = wl[2] - sx, segy = wl[3] - sy;
      float offx = sx - v->x, offy = sy - v->y;
      float den = rx * segy - ry * segx;
      int small = fabsf(den) < 1e-6f;
      float safe = small ? 1.0f : den;
      float distance = (offx * segy - offy * segx) / safe;
      float al = (offx * ry - offy * rx) / safe;
      int valid = !small && distance > 0 && al >= 0 && al <= 1;
      float d = valid ? distance : INFINITY;
      if (d < best) { best = d; bestSlot = b; }
    }
    g->blockingWall[x] = sc->blocking[bestSlot];
    g->wallDistance[x] = fminf(fmaxf(best, 1.0f), 4096.0f);
  }
}

/* PrepWall for one (column, wall) (engine.py:10672-10739). */
static void prep_wall(const Scene *sc, const WallView *wv, int w, int x, i64 *hoff, i64 *vstep) {
  i64 tx1 = wv->tx[0], tx2 = wv->tx[1], ty1 = wv->ty[0], ty2 = wv->ty[1];
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
  i64 repeat = rint_f(sc->wlen[w] * 65536.0f);
  *hoff = (i64)floor(fraction * (double)repeat + 0.5);
  double wms = (320 * 200.0 / 320.0 / 240) * 64.0 / (320 / 2.0);
  double depthScale = (double)(invzStepF * (float)wms);
  double depthOrigin = (double)((-(float)uozStep) * (float)wms);
  *vstep = (i64)floor(fraction * depthScale + depthOrigin + 0.5);
}

/* OWallMost row projection (engine.py:12294-12605), single-fragment walls. */
/* The unclipped whole-line projection: what a column of a split line falls back to when none of
 * the line's fragments owns it (engine.py:12393-12410, 12596-12604). */
static i64 project_rows_whole(const View *v, const WallView *wv, float worldZ, int x) {
  i64 wsl = wv->sl, wsr = wv->sr;
  i64 wdl = imax(wv->dl, 1), wdr = imax(wv->dr, 1);
  i64 relZ = rint_f((worldZ - v->viewZ) * 65536.0f);
  i64 pz = -(relZ >> 4);
  i64 ospan = imax(wsr - wsl, 1);
  i64 opl = (pz * FOCAL_Y) / wdl, opr = (pz * FOCAL_Y) / wdr;
  i64 ostep = (opr - opl) / ospan;
  return iclamp((v->center + opl + (x - wsl) * ostep) >> 16, 0, VH);
}

static i64 project_rows(const View *v, const WallView *wv, float worldZ, int x);

/* Which FWallCoords the row projection and the wallscan light of line w use at column x: the
 * line itself, or, for a split line, the first of its fragments whose span holds the column
 * (engine.py:12310-12376, 11511-11545); NULL when the line is split and no fragment does. */
static const WallView *projection_fragment(const Scene *sc, const LaneGeom *g, int w, int x) {
  int f0 = sc->fragOff[w], f1 = sc->fragOff[w + 1];
  if (sc->F <= 0 || f1 <= f0) return &g->wv[w];
  for (int f = f0; f < f1; ++f) {
    const WallView *q = &g->frag[f];
    if (q->sr > q->sl && x >= q->sl && x < q->sr) return q;
  }
  return NULL;
}

static i64 line_rows(const Scene *sc, const View *v, const LaneGeom *g, int w, float worldZ, int x) {
  const WallView *q = projection_fragment(sc, g, w, x);
  return q ? project_rows(v, q, worldZ, x) : project_rows_whole(v, &g->wv[w], worldZ, x);
}

static i64 line_vis(const Scene *sc, const LaneGeom *g, int w, int side, int x) {
  const WallView *q = projection_fragment(sc, g, w, x);
  if (!q) q = &g->wv[w];
  return q->visL[side] + ((i64)x - q->visSl[side]) * q->visStep[side];
}

static i64 project_rows(const View *v, const WallView *wv, float worldZ, int x) {
  i64 wsl = wv->sl, wsr = wv->sr;
  i64 wdl = imax(wv->dl, 1), wdr = imax(wv->dr, 1);
  int owns = (wsr > wsl) && x >= wsl && x < wsr;
  i64 sl = wsl, sr = wsr, dl = wdl, dr = wdr;
  i64 relZ = rint_f((worldZ - v->viewZ) * 65536.0f);
  i64 pz = -(relZ >> 4);
  i64 center = v->center;
  i64 ospan = imax(wsr - wsl, 1);
  i64 opl = (pz * FOCAL_Y) / wdl, opr = (pz * FOCAL_Y) / wdr;
  i64 ostep = (opr - opl) / ospan;
  i64 original = iclamp((center + opl + (x - wsl) * ostep) >> 16, 0, VH);
  if (!owns) return original;
  i64 upperClip = ((-center) * FU) / FOCAL_Y;
  i64 lowerClip = ((VH * FU - center) * FU) / FOCAL_Y;
  i64 ul = (upperClip * dl) >> 16, ur = (upperClip * dr) >> 16;
  i64 ll = (lowerClip * dl) >> 16, lr = (lowerClip * dr) >> 16;
  int aboveL = pz < ul, aboveR = pz < ur, belowL = pz > ll, belowR = pz > lr;
  int entAbove = aboveL && aboveR, entBelow = belowL && belowR;
  i64 cl = sl, cr = sr, cdl = dl, cdr = dr;
  int outTop = 0, outBottom = 0;
  int crossesTop = aboveL ^ aboveR;
  i64 sud = (ur != ul) ? (ur - ul) : 1;
  i64 tf = shl(pz - ul, 30) / sud;
  i64 td = dl + (((dr - dl) * tf) >> 30);
  i64 tc = sl + ((((dr * tf) >> 30)) * (sr - sl)) / imax(td, 1);
  int ctr = crossesTop && aboveR && (sl <= tc);
  if (ctr) { cr = tc; cdr = td; }
  outTop |= crossesTop && aboveR && (sr > tc) && (x >= tc) && (x < sr);
  int ctl = crossesTop && aboveL && (tc <= sr);
  if (ctl) { cl = tc; cdl = td; }
  outTop |= crossesTop && aboveL && (tc > sl) && (x >= sl) && (x < tc);
  int crossesBottom = belowL ^ belowR;
  i64 sld = (lr != ll) ? (lr - ll) : 1;
  i64 bf = shl(pz - ll, 30) / sld;
  i64 bd = dl + (((dr - dl) * bf) >> 30);
  i64 bc = sl + ((((dr * bf) >> 30)) * (sr - sl)) / imax(bd, 1);
  int cbr = crossesBottom && belowR && (sl <= bc);
  if (cbr) { cr = bc; cdr = bd; }
  outBottom |= crossesBottom && belowR && (sr > bc) && (x >= bc) && (x < sr);
  int cbl = crossesBottom && belowL && (bc <= sr);
  if (cbl) { cl = bc; cdl = bd; }
  outBottom |= crossesBottom && belowL && (bc > sl) && (x >= sl) && (x < bc);
  i64 pl = (pz * FOCAL_Y) / imax(cdl, 1), pr = (pz * FOCAL_Y) / imax(cdr, 1);
  i64 span = imax(cr - cl, 1);
  i64 pstep = (pr - pl) / span;
  i64 projected = iclamp((center + pl + (x - cl) * pstep) >> 16, 0, VH);
  int collapsed = (cr == cl) && (x == cl) && !(entAbove || entBelow);
  if (entAbove || (outTop && !collapsed)) projected = 0;
  else if (entBelow || (outBottom && !collapsed)) projected = VH;
  return projected;
}

static inline int wall_shade(i64 light, i64 vis) {
  i64 base = 64 * FU - (light + 12) * (FU / 4);
  return (int)iclamp((base - imin(vis, 24 * FU)) >> 16, 0, 31);
}

typedef struct {
  float depth[VH * SW];   /* sprite_clip_depth */
  int32_t wall[VH * SW];  /* sprite_clip_wall */
} SpriteClip;

typedef struct {
  int cur;
  i64 ceilClip, floorClip;
  float prev;
  int pendOwnerBoundary; float pendOwnerEp[2];
  int pendEpBoundary; float pendEpEp[2]; int pendEpWall;
  int pendEpBridgeBoundary, pendEpBridgeIndex;
  int pendPortalBridge, pendPortalBridgeIndex, pendPortalBridgeSector; float pendPortalBridgeExit;
} ColState;

typedef struct {
  int wall, side;
  int rasterValid, valid;
  int oneSided;
  int renderCurrent, safeOther, otherSector;
  float distance;
  i64 vis;
  i64 ctop, cbot, cupbot, clowtop;   /* clipped rows */
  int tier[3];
  int markCeil, markFloor;
  float viewFloor, viewCeil, otherFloor, otherCeil;
  int tex[3];
  /* decisions carried into the traversal update */
} ColIter;

static inline int secidx(const Scene *sc, int s) { return s < 0 ? s + sc->S : s; }
static inline float sec_floor(const Scene *sc, int s) { return sc->secF[secidx(sc, s) * 2]; }
static inline float sec_ceil(const Scene *sc, int s) { return sc->secF[secidx(sc, s) * 2 + 1]; }
static inline int sec_light(const Scene *sc, int s) { return sc->secI[secidx(sc, s) * 4]; }
static inline int sec_ftex(const Scene *sc, int s) { return sc->secI[secidx(sc, s) * 4 + 1]; }
static inline int sec_ctex(const Scene *sc, int s) { return sc->secI[secidx(sc, s) * 4 + 2]; }

static inline int same_pair(const Scene *sc, int a, int b) {
  const int32_t *A = &sc->wsec[a * 2], *B = &sc->wsec[b * 2];
  return (A[0] == B[0] && A[1] == B[1]) || (A[0] == B[1] && A[1] == B[0]);
}
static inline int shares_any_endpoint(const Scene *sc, int a, int b) {
  const int32_t *A = &sc->wvtx[a * 2], *B = &sc->wvtx[b * 2];
  return A[0] == B[0] || A[0] == B[1] || A[1] == B[0] || A[1] == B[1];
}
/* engine.py:1605-1612 */
static int opposing_pair(const Scene *sc, int a, int b) {
  if (!same_pair(sc, a, b)) return 0;
  if (sc->wsec[a * 2 + 1] < 0 || sc->wsec[b * 2 + 1] < 0) return 0;
  if (shares_any_endpoint(sc, a, b)) return 0;
  const float *A = &sc->walls[a * 4], *B = &sc->walls[b * 4];
  float adx = A[2] - A[0], ady = A[3] - A[1], bdx = B[2] - B[0], bdy = B[3] - B[1];
  float dot = adx * bdx + ady * bdy;
  float cross = adx * bdy - ady * bdx;
  return dot < 0 && fabsf(cross) < 1e-6f;
}
static inline int two_distinct(const Scene *sc, int w) {
  return sc->wsec[w * 2 + 1] >= 0 && sc->wsec[w * 2] != sc->wsec[w * 2 + 1];
}
/* sector set of wall c equals the symmetric difference of the sets of a and b
 * (a and b two-sided with distinct sectors sharing exactly one). */
static int bridge_pair_of(const Scene *sc, int a, int b, int *p0, int *p1) {
  int a0 = sc->wsec[a * 2], a1 = sc->wsec[a * 2 + 1], b0 = sc->wsec[b * 2], b1 = sc->wsec[b * 2 + 1];
  int shared = 0, sv = -2;
  if (a0 == b0 || a0 == b1) { shared++; sv = a0; }
  if (a1 == b0 || a1 == b1) { shared++; sv = a1; }
  if (shared != 1) return 0;
  *p0 = (a0 == sv) ? a1 : a0;
  *p1 = (b0 == sv) ? b1 : b0;
  return 1;
}
static int set_equals(const Scene *sc, int w, int p0, int p1) {
  int s0 = sc->wsec[w * 2], s1 = sc->wsec[w * 2 + 1];
  if (p0 == p1) return s0 == p0 && s1 == p0;
  return (s0 == p0 && s1 == p1) || (s0 == p1 && s1 == p0);
}
/* engine.py:399-440: bridge at endpoint `slot` of `path` for `owner`. */
static int portal_bridge(const Scene *sc, int slot, int path, int owner, int *index) {
  *index = 0;
  if (!two_distinct(sc, path)) return 0;
  if (owner == path) return 0;
  int v = sc->wvtx[path * 2 + slot];
  const int32_t *ov = &sc->wvtx[owner * 2];
  if (ov[0] != v && ov[1] != v) return 0;
  if (!two_distinct(sc, owner)) return 0;
  int p0, p1;
  if (!bridge_pair_of(sc, path, owner, &p0, &p1)) return 0;
  int count = 0, found = 0;
  for (int k = sc->vtxOff[v]; k < sc->vtxOff[v + 1]; ++k) {
    int c = sc->vtxWalls[k];
    if (c == path || c == owner) continue;
    if (set_equals(sc, c, p0, p1)) { count++; found = c; }
  }
  if (count == 1) { *index = found; return 1; }
  return 0;
}
/* engine.py:443-484: bridge at endpoint `slot` of `pending` for any `path`. */
static int sector_bridge(const Scene *sc, int slot, int pending, int path, int *index) {
  *index = 0;
  if (!two_distinct(sc, pending)) return 0;
  if (path == pending) return 0;
  if (!two_distinct(sc, path)) return 0;
  int p0, p1;
  if (!bridge_pair_of(sc, pending, path, &p0, &p1)) return 0;
  int v = sc->wvtx[pending * 2 + slot];
  int count = 0, found = 0;
  for (int k = sc->vtxOff[v]; k < sc->vtxOff[v + 1]; ++k) {
    int c = sc->vtxWalls[k];
    if (c == pending || c == path) continue;
    if (set_equals(sc, c, p0, p1)) { count++; found = c; }
  }
  if (count == 1) { *index = found; return 1; }
  return 0;
}

typedef struct {
  uint8_t frame[VH * SW];
  uint8_t filled[VH * SW];
  int16_t planeSector[VH * SW];
  uint8_t planeIsFloor[VH * SW];
  /* depth of the surface every pixel shows (engine.py:11551-11553, 12872, 13412, 13740): what a
   * decal is tested against */
  float sceneDepth[VH * SW];
  SpriteClip clip;
  /* nearest raster-valid two-sided crossing with a middle texture, per column
   * (engine.py:11573-11579, 12914-12939) */
  int maskedWall[SW];
  i64 maskedCeil[SW], maskedFloor[SW];
  float maskedDist[SW];
} LaneBuffers;

static void wall_pass(const Scene *sc, const View *v, const LaneGeom *g, LaneBuffers *lb) {
  int W = sc->W;
  ColState *cs = calloc(SW, sizeof(ColState));
  ColIter *ci = calloc(SW, sizeof(ColIter));
  memset(lb->filled, 0, sizeof lb->filled);
  memset(lb->planeIsFloor, 0, sizeof lb->planeIsFloor);
  for (int i = 0; i < VH * SW; ++i) {
    lb->planeSector[i] = -1;
    lb->clip.depth[i] = INFINITY;
    lb->clip.wall[i] = -1;
  }
  /* current sector of the viewer (engine.py:9598-9620) */
  int startSector = 0;
  {
    for (int s = 0; s < sc->S; ++s) {
      int crossings = 0;
      for (int k = sc->edgeOff[s]; k < sc->edgeOff[s + 1]; ++k) {
        const float *e = &sc->walls[sc->edgeWalls[k] * 4];
        float x1 = e[0], y1 = e[1], x2 = e[2], y2 = e[3];
        int crosses = (y1 > v->y) != (y2 > v->y);
        float dy = y2 - y1;
        float safe = fabsf(dy) < 1e-6f ? 1.0f : dy;
        float cx = x1 + (v->y - y1) * (x2 - x1) / safe;
        crossings += crosses && (v->x < cx);
      }
      if (crossings & 1) { startSector = s; break; }
    }
  }
  for (int x = 0; x < SW; ++x) {
    lb->maskedWall[x] = -1;
    lb->maskedCeil[x] = 0;
    lb->maskedFloor[x] = VH;
    lb->maskedDist[x] = INFINITY;
    cs[x].cur = startSector;
    cs[x].ceilClip = 0;
    cs[x].floorClip = VH;
    cs[x].prev = 0.0f;
    cs[x].pendPortalBridgeSector = -1;
  }

  for (int iter = 0; iter < sc->S; ++iter) {
    int anyAlive = 0;
    for (int x = 0; x < SW; ++x) anyAlive |= cs[x].cur >= 0;
    if (!anyAlive) break;
    /* decisions saved for the traversal update of each column */
    typedef struct {
      int nokpp, pskpp, usesGeo, entersOther, entersShared, endpointOnly, epb, cppb, geometric;
      int nopOther, psOther, gpOther;
      float nopDist, psDist, gpDist, osd;
      int startsOwner, continuesOwner;
      float selEp[2], epEp[2];
      int pendEpHasFwd, epFwdIdx, ppbIdx;
      int psPathIndex, psFromFront;
    } Trav;
    Trav *trav = calloc(SW, sizeof(Trav));
    for (int x = 0; x < SW; ++x) {
      ColState *c = &cs[x];
      ColIter *it = &ci[x];
      Trav *t = &trav[x];
      memset(it, 0, sizeof *it);
      memset(t, 0, sizeof *t);
      const float *D = &g->dist[x * W];
      const float *AL = &g->along[x * W];
      const uint8_t *G = &g->geo[x * W], *PJ = &g->proj[x * W], *LE = &g->left[x * W];
      int curSector = c->cur;
      int current = curSector < 0 ? 0 : curSector;
      float prev = c->prev;
#define INCIDENT(w) (sc->wsec[(w) * 2] == current || sc->wsec[(w) * 2 + 1] == current)
#define TOL(w) fmaxf(fabsf(D[w]) / 128.0f, 4.0f)
      float distance = INFINITY;
      int wallIndex = 0;
      for (int w = 0; w < W; ++w) {
        if (INCIDENT(w) && curSector >= 0 && D[w] > prev && D[w] < distance) { distance = D[w]; wallIndex = w; }
      }
      {
        float sd = INFINITY;
        int sw = 0;
        for (int w = 0; w < W; ++w) {
          int cand = INCIDENT(w) && curSector >= 0 && D[w] > prev;
          if (!cand || !isfinite(D[w])) continue;
          if (g->wv[w].oneSided && fabsf(D[w] - distance) <= 1e-3f && D[w] < sd) { sd = D[w]; sw = w; }
        }
        if (isfinite(sd)) { distance = sd; wallIndex = sw; }
      }
      float selAlong = AL[wallIndex];
      const float *selWall = &sc->walls[wallIndex * 4];
      int selUsesStart = selAlong <= 0.5f;
      float selEp[2] = {selUsesStart ? selWall[0] : selWall[2], selUsesStart ? selWall[1] : selWall[3]};
      int selVtx = sc->wvtx[wallIndex * 2 + (selUsesStart ? 0 : 1)];
#define SHARES_SEL(w) (sc->wvtx[(w) * 2] == selVtx || sc->wvtx[(w) * 2 + 1] == selVtx)
      int continuesOwner = c->pendOwnerBoundary && selEp[0] == c->pendOwnerEp[0] && selEp[1] == c->pendOwnerEp[1];
      int continuesEp = c->pendEpBoundary && selEp[0] == c->pendEpEp[0] && selEp[1] == c->pendEpEp[1];
      int selSlot = selAlong > 0.5f;
      int epFwdIdx;
      int epFwdMask = portal_bridge(sc, selSlot, wallIndex, c->pendEpWall, &epFwdIdx);
      int pendEpHasFwd = continuesEp && epFwdMask && (D[epFwdIdx] > distance + 1e-3f);
      int completesPendEpBridge = c->pendEpBridgeBoundary && wallIndex == c->pendEpBridgeIndex;
      int selIsProjected = PJ[wallIndex];
      int selExclRight = g->wv[wallIndex].sr == x;
      float psPathDist = distance;
      int psPathIndex = wallIndex;
      float psd = INFINITY;
      int psi = 0;
      for (int w = 0; w < W; ++w) {
        int owner = INCIDENT(w) && g->wv[w].oneSided && PJ[w] && LE[w] && SHARES_SEL(w) && !selIsProjected &&
                    (D[w] > prev + 1e-3f);
        if (owner && D[w] < psd) { psd = D[w]; psi = w; }
      }
      {
        const int32_t *off = selUsesStart ? sc->sbStartOff : sc->sbEndOff;
        const int32_t *idx = selUsesStart ? sc->sbStartIdx : sc->sbEndIdx;
        float sbd = INFINITY;
        int sbi = wallIndex;
        int first = 1;
        for (int k = off[wallIndex]; k < off[wallIndex + 1]; ++k) {
          int b = idx[k];
          if (first) { sbi = b; first = 0; }
          int owner = selExclRight && INCIDENT(b) && g->wv[b].oneSided && PJ[b] && LE[b] && !selIsProjected &&
                      (D[b] > prev + 1e-3f);
          if (owner && D[b] < sbd) { sbd = D[b]; sbi = b; }
        }
        if (sbd < psd) { psd = sbd; psi = sbi; }
      }
      int hasProjectedSolidOwner = isfinite(psd);
      if (hasProjectedSolidOwner) { distance = psd; wallIndex = psi; }
      int seo = g->eoIdx[x * W + wallIndex];
      float sed = g->eoDist[x * W + wallIndex];
      int eoPathIsGeo = G[wallIndex];
      int replaceEo = (seo != wallIndex) && (sed > prev + 1e-3f);
      if (replaceEo) { distance = sed; wallIndex = seo; }
      int nopIndex = wallIndex;
      float nopDist = distance;
      int nopIsGeo = replaceEo ? eoPathIsGeo : G[wallIndex];
      int nopFromFront = curSector == sc->wsec[nopIndex * 2];
      int nopOther = nopFromFront ? sc->wsec[nopIndex * 2 + 1] : sc->wsec[nopIndex * 2];
      int selOwnerIsProjected = PJ[wallIndex];
      int selOwnerExclRight = g->wv[wallIndex].sr == x;
      i64 selOwnerSpan = g->wv[wallIndex].sr - g->wv[wallIndex].sl;
      int selOwnerShort = sc->wlen[wallIndex] <= 32.0f;
      float npd = INFINITY;
      int npi = 0;
      for (int w = 0; w < W; ++w) {
        if (!(INCIDENT(w) && !g->wv[w].oneSided && PJ[w])) continue;
        if (selOwnerIsProjected || !(D[w] > prev + 1e-3f)) continue;
        int sbIdx;
        int candHasSectorBridge = sector_bridge(sc, AL[w] > 0.5f, w, nopIndex, &sbIdx);
        int topological = LE[w] && selOwnerExclRight && selOwnerSpan <= 2 && candHasSectorBridge;
        int a = same_pair(sc, wallIndex, w) ||
                (LE[w] && selOwnerExclRight && (selOwnerSpan <= 2 || (SHARES_SEL(w) && selOwnerShort)));
        int near = (a && (fabsf(D[w] - distance) <= TOL(w))) || topological;
        if (near && D[w] < npd) { npd = D[w]; npi = w; }
      }
      /* projected sector bridge (engine.py:12073-12164) */
      int pew = c->pendEpWall;
      int peFromCur = curSector == sc->wsec[pew * 2];
      int peIncident = peFromCur || curSector == sc->wsec[pew * 2 + 1];
      int peOther = peFromCur ? sc->wsec[pew * 2 + 1] : sc->wsec[pew * 2];
      const float *peWall = &sc->walls[pew * 4];
      int peSlot = (c->pendEpEp[0] == peWall[2] && c->pendEpEp[1] == peWall[3]) ? 1 : 0;
      int psbIndex;
      int psbExists = sector_bridge(sc, peSlot, pew, nopIndex, &psbIndex);
      int b0 = sc->wsec[psbIndex * 2], b1 = sc->wsec[psbIndex * 2 + 1];
      int psbMatches = (b0 == peOther && b1 == nopOther) || (b1 == peOther && b0 == nopOther);
      float psbDist = D[psbIndex];
      int psb = c->pendEpBoundary && peIncident && peOther >= 0 && nopOther >= 0 &&
                (g->wv[pew].sr - g->wv[pew].sl <= 1) && nopIsGeo && !selOwnerIsProjected && selOwnerExclRight &&
                psbExists && psbMatches && PJ[psbIndex] && LE[psbIndex] && (psbDist > prev - TOL(pew)) &&
                (psbDist < nopDist);
      if (!psb) psbDist = INFINITY;
      int usePsb = psbDist < npd;
      if (usePsb) { npd = psbDist; npi = psbIndex; }
      int replaceNp = isfinite(npd);
      int startsOwner = replaceNp;
      if (replaceNp) { distance = npd; wallIndex = npi; }
      int finalIsProjected = PJ[wallIndex], finalIsGeo = G[wallIndex];
      int completesOpposing = c->pendEpBoundary && opposing_pair(sc, pew, wallIndex) && finalIsProjected && !finalIsGeo;
      int valid = isfinite(distance);
      int exclTraversalOnly = !selOwnerIsProjected && selOwnerExclRight && !replaceNp && selOwnerSpan <= 2 &&
                              !g->boundaryHasProjectedOwner[x];
      int rasterValid = valid && !exclTraversalOnly && !continuesOwner &&
                        !((pendEpHasFwd || completesPendEpBridge) && !selIsProjected && selExclRight && !replaceNp);
      int geometric = replaceNp ? nopIsGeo : (replaceEo ? eoPathIsGeo : G[wallIndex]);
      int nokpp = replaceNp && nopIsGeo && nopOther >= 0;
      int front = sc->wsec[wallIndex * 2], back = sc->wsec[wallIndex * 2 + 1];
      int fromFront = curSector == front;
      int otherSector = fromFront ? back : front;
      int renderCurrent = usePsb ? peOther : (completesOpposing ? otherSector : current);
      int renderFromFront = renderCurrent == front;
      int renderOther = renderFromFront ? back : front;
      int side = !renderFromFront;
      const WallView *wv = &g->wv[wallIndex];
      i64 vis = line_vis(sc, g, wallIndex, side, x);
      int psFromFront = curSector == sc->wsec[psPathIndex * 2];
      int psOther = psFromFront ? sc->wsec[psPathIndex * 2 + 1] : sc->wsec[psPathIndex * 2];
      int psIsGeo = G[psPathIndex];
      int pskpp = hasProjectedSolidOwner && psIsGeo && psOther >= 0;
      int safeOther = renderOther < 0 ? 0 : renderOther;
      float viewFloor = sec_floor(sc, renderCurrent), viewCeil = sec_ceil(sc, renderCurrent);
      float otherFloor = sec_floor(sc, safeOther), otherCeil = sec_ceil(sc, safeOther);
      int oneSided = otherSector < 0;
      const int32_t *stex = &sc->sideTex[(wallIndex * 2 + side) * 3];
      i64 oneTop = line_rows(sc, v, g, wallIndex, viewCeil, x), oneBottom = line_rows(sc, v, g, wallIndex, viewFloor, x);
      i64 lowerTop = line_rows(sc, v, g, wallIndex, otherFloor, x), upperBottom = line_rows(sc, v, g, wallIndex, otherCeil, x);
      i64 ctop = imax(oneTop, c->ceilClip), cbot = imin(oneBottom, c->floorClip);
      i64 cupbot = imax(imin(upperBottom, c->floorClip), ctop);
      i64 clowtop = imin(imax(lowerTop, c->ceilClip), cbot);
      int lightDiff = sec_light(sc, renderCurrent) != sec_light(sc, safeOther);
      int markCeil = oneSided || viewCeil != otherCeil || sec_ctex(sc, renderCurrent) != sec_ctex(sc, safeOther) || lightDiff;
      int markFloor = oneSided || viewFloor != otherFloor || sec_ftex(sc, renderCurrent) != sec_ftex(sc, safeOther) || lightDiff;
      /* plane marks */
      if (rasterValid) {
        i64 cpb = imin(ctop, c->floorClip), fpt = imax(cbot, c->ceilClip);
        if (markFloor)
          for (i64 y = fpt; y < c->floorClip; ++y)
            if (lb->planeSector[y * SW + x] < 0) { lb->planeSector[y * SW + x] = (int16_t)renderCurrent; lb->planeIsFloor[y * SW + x] = 1; }
        if (markCeil)
          for (i64 y = c->ceilClip; y < cpb; ++y)
            if (lb->planeSector[y * SW + x] < 0) lb->planeSector[y * SW + x] = (int16_t)renderCurrent;
      }
      it->wall = wallIndex; it->side = side; it->rasterValid = rasterValid; it->valid = valid;
      it->oneSided = oneSided; it->renderCurrent = renderCurrent; it->safeOther = safeOther; it->otherSector = otherSector;
      it->distance = distance; it->vis = vis;
      it->ctop = ctop; it->cbot = cbot; it->cupbot = cupbot; it->clowtop = clowtop;
      it->viewFloor = viewFloor; it->viewCeil = viewCeil; it->otherFloor = otherFloor; it->otherCeil = otherCeil;
      it->tex[0] = stex[0]; it->tex[1] = stex[1]; it->tex[2] = stex[2];
      it->markCeil = markCeil; it->markFloor = markFloor;
      it->tier[0] = oneSided && rasterValid && stex[0] >= 0 && ctop < cbot;
      it->tier[1] = !oneSided && rasterValid && (viewFloor < otherFloor) && stex[1] >= 0 && clowtop < cbot;
      it->tier[2] = !oneSided && rasterValid && (viewCeil > otherCeil) && stex[2] >= 0 && ctop < cupbot;

      /* traversal bookkeeping that only needs this column's data */
      float cnd = INFINITY, ond = INFINITY; int cni = 0, oni = 0;
      float csd = INFINITY, osd = INFINITY;
      float gpd = INFINITY; int gpi = 0;
      float prior = prev;
      for (int w = 0; w < W; ++w) {
        int inc = INCIDENT(w);
        int oinc = sc->wsec[w * 2] == otherSector || sc->wsec[w * 2 + 1] == otherSector;
        int os = g->wv[w].oneSided;
        int fut = (G[w] || (os && isfinite(D[w]))) && (D[w] > distance + 1e-3f);
        if (inc && fut && D[w] < cnd) { cnd = D[w]; cni = w; }
        if (oinc && fut && D[w] < ond) { ond = D[w]; oni = w; }
        int sharesEp = shares_any_endpoint(sc, w, wallIndex);
        int sharedSolid = isfinite(D[w]) && os && (sharesEp || LE[w]) && (D[w] > prior + 1e-3f) && (D[w] <= distance + 1e-3f);
        if (inc && sharedSolid && D[w] < csd) csd = D[w];
        if (oinc && sharedSolid && D[w] < osd) osd = D[w];
        int sgp = G[w] && inc && sharesEp && !os && (D[w] > prior + 1e-3f) && (fabsf(D[w] - distance) <= (1.0f / 16.0f));
        if (sgp && D[w] < gpd) { gpd = D[w]; gpi = w; }
      }
      int endpointOnly = valid && !oneSided && !geometric;
      int tied = endpointOnly && isfinite(cnd) && cni == oni && opposing_pair(sc, wallIndex, cni);
      int entersOther = endpointOnly && otherSector >= 0 && ((ond < cnd) || tied);
      int entersShared = endpointOnly && otherSector >= 0 && (osd < csd);
      int gpFromFront = curSector == sc->wsec[gpi * 2];
      int gpOther = gpFromFront ? sc->wsec[gpi * 2 + 1] : sc->wsec[gpi * 2];
      int usesGeo = endpointOnly && isfinite(gpd) && gpOther >= 0;
      int pbSlot = AL[gpi] > 0.5f;
      int ppbIdx;
      int ppbExists = portal_bridge(sc, pbSlot, gpi, wallIndex, &ppbIdx);
      float ppbDist = D[ppbIdx];
      int epb = usesGeo && ppbExists && PJ[ppbIdx] && LE[ppbIdx] && (ppbDist > prior + 1e-3f) &&
                (fabsf(ppbDist - gpd) <= TOL(gpi));
      int cppb = valid && c->pendPortalBridge && wallIndex == c->pendPortalBridgeIndex;
      t->nokpp = nokpp; t->pskpp = pskpp; t->usesGeo = usesGeo; t->entersOther = entersOther;
      t->entersShared = entersShared; t->endpointOnly = endpointOnly; t->epb = epb; t->cppb = cppb;
      t->geometric = geometric;
      t->nopOther = nopOther; t->psOther = psOther; t->gpOther = gpOther;
      t->nopDist = nopDist; t->psDist = psPathDist; t->gpDist = gpd; t->osd = osd;
      t->startsOwner = startsOwner; t->continuesOwner = continuesOwner;
      t->selEp[0] = selEp[0]; t->selEp[1] = selEp[1];
      {
        const float *fw = &sc->walls[wallIndex * 4];
        int us = AL[wallIndex] <= 0.5f;
        t->epEp[0] = us ? fw[0] : fw[2];
        t->epEp[1] = us ? fw[1] : fw[3];
      }
      t->pendEpHasFwd = pendEpHasFwd; t->epFwdIdx = epFwdIdx; t->ppbIdx = ppbIdx;
      t->psPathIndex = psPathIndex; t->psFromFront = psFromFront;
#undef INCIDENT
#undef TOL
#undef SHARES_SEL
    }

    /* aligned 4-column wallscan groups (engine.py:12694-12761) */
    for (int gx = 0; gx < SW; gx += 4) {
      int same = 1;
      for (int k = 1; k < 4; ++k) same &= (ci[gx + k].wall == ci[gx].wall) && (ci[gx + k].side == ci[gx].side);
      i64 groupBottom[3];
      int groupValid[3];
      for (int tier = 0; tier < 3; ++tier) {
        i64 ctopMax = -1, cbotMin = 1 << 20;
        int all = 1;
        for (int k = 0; k < 4; ++k) {
          const ColIter *it = &ci[gx + k];
          i64 top = tier == 1 ? it->clowtop : it->ctop;
          i64 bot = tier == 2 ? it->cupbot : it->cbot;
          ctopMax = imax(ctopMax, top);
          cbotMin = imin(cbotMin, bot);
          all &= it->tier[tier];
        }
        groupValid[tier] = same && all && ctopMax < cbotMin;
        groupBottom[tier] = cbotMin;
      }
      i64 firstVis = ci[gx].vis;
      for (int k = 0; k < 4; ++k) {
        int x = gx + k;
        ColState *c = &cs[x];
        ColIter *it = &ci[x];
        const Trav *t = &trav[x];
        int wallIndex = it->wall, side = it->side;
        const WallView *wv = &g->wv[wallIndex];
        if (it->rasterValid) {
          i64 hoff, vstepBase;
          prep_wall(sc, wv, wallIndex, x, &hoff, &vstepBase);
          i64 repeat = rint_f(sc->wlen[wallIndex] * 65536.0f);
          if (side != 0) hoff = repeat - hoff;
          if (wv->sl > 0 && hoff < 0) hoff = 0;
          if (hoff >= repeat) hoff = repeat - 1;
          const float *soff = &sc->sideOff[(wallIndex * 2 + side) * 2];
          i64 tox = rint_f(soff[0] * 65536.0f);
          const float *wl = &sc->walls[wallIndex * 4];
          int horizontal = fabsf(wl[3] - wl[1]) < 1e-6f, vertical = fabsf(wl[2] - wl[0]) < 1e-6f;
          i64 light = sec_light(sc, it->renderCurrent) + v->flashLight * 16 + (vertical ? 16 : (horizontal ? -16 : 0));
          int oneSided = it->oneSided;
          for (int y = 0; y < VH; ++y) {
            int oneSpan = oneSided && y >= it->ctop && y < it->cbot;
            int lowerSpan = !oneSided && (it->viewFloor < it->otherFloor) && y >= it->clowtop && y < it->cbot;
            int upperSpan = !oneSided && (it->viewCeil > it->otherCeil) && y >= it->ctop && y < it->cupbot;
            if (!(oneSpan || lowerSpan || upperSpan)) continue;
            int texId = oneSpan ? it->tex[0] : (lowerSpan ? it->tex[1] : it->tex[2]);
            if (texId < 0 || lb->filled[y * SW + x]) continue;
            float originZ = oneSpan ? it->viewCeil : (lowerSpan ? it->otherFloor : it->otherCeil);
            const int32_t *ti = &sc->texInfo[texId * 4];
            int tw = ti[0], hbits = ti[3];
            i64 u = pymod((hoff + tox) >> 16, tw);
            i64 vstep = vstepBase * (1LL << (14 - hbits));
            i64 screenDelta = (i64)y * FU - v->center + FU;
            i64 texMid = rint_f((originZ - v->viewZ) * 65536.0f + soff[1] * 65536.0f);
            i64 frac = shl(texMid, 16 - hbits) + (wrap_mul(vstep, screenDelta) >> 16);
            i64 tv = (frac & U32MASK) >> (32 - hbits);
            uint8_t texel = sc->texAtlas[((size_t)texId * sc->texH + tv) * sc->texW + u];
            int tail = (oneSpan && groupValid[0] && y >= groupBottom[0]) ||
                       (lowerSpan && groupValid[1] && y >= groupBottom[1]) ||
                       (upperSpan && groupValid[2] && y >= groupBottom[2]);
            int shade = wall_shade(light, tail ? firstVis : it->vis);
            lb->frame[y * SW + x] = sc->colormap[shade * 256 + texel];
            lb->filled[y * SW + x] = 1;
            lb->sceneDepth[y * SW + x] = it->distance;
            if (it->distance < lb->clip.depth[y * SW + x]) {
              lb->clip.depth[y * SW + x] = it->distance;
              lb->clip.wall[y * SW + x] = wallIndex;
            }
          }
        }
        /* clip updates (engine.py:12885-12913) */
        int hasUpper = it->tex[2] >= 0, hasLower = it->tex[1] >= 0;
        int drawsUpper = (it->viewCeil > it->otherCeil) && hasUpper;
        int drawsLower = (it->viewFloor < it->otherFloor) && hasLower;
        if (it->rasterValid && !it->oneSided && (drawsUpper || it->markCeil)) c->ceilClip = drawsUpper ? it->cupbot : it->ctop;
        if (it->rasterValid && !it->oneSided && (drawsLower || it->markFloor)) c->floorClip = drawsLower ? it->clowtop : it->cbot;
        /* masked drawseg snapshot (engine.py:12914-12939) */
        if (it->rasterValid && !it->oneSided && it->tex[0] >= 0 && it->distance < lb->maskedDist[x]) {
          lb->maskedCeil[x] = c->ceilClip;
          lb->maskedFloor[x] = c->floorClip;
          lb->maskedDist[x] = it->distance;
          lb->maskedWall[x] = wallIndex;
        }
        /* sprite silhouettes (engine.py:12940-12964) */
        int masked = it->tex[0] >= 0;
        int bottomSil = !it->oneSided && ((it->viewFloor > it->otherFloor) || (v->viewZ < it->otherFloor) || masked);
        int topSil = !it->oneSided && ((it->viewCeil < it->otherCeil) || (v->viewZ > it->otherCeil) || masked);
        if (it->rasterValid) {
          for (int y = 0; y < VH; ++y) {
            int in = (bottomSil && y >= c->floorClip) || (topSil && y < c->ceilClip);
            if (in && it->distance < lb->clip.depth[y * SW + x]) {
              lb->clip.depth[y * SW + x] = it->distance;
              lb->clip.wall[y * SW + x] = wallIndex;
            }
          }
        }
        /* clips contributed by the crossed portal behind a projected solid
         * (engine.py:12965-13069) */
        if (t->pskpp) {
          int pIdx = t->psPathIndex;
          const WallView *pw = &g->wv[pIdx];
          int pSafeOther = t->psOther < 0 ? 0 : t->psOther;
          float pOtherFloor = sec_floor(sc, pSafeOther), pOtherCeil = sec_ceil(sc, pSafeOther);
          int pSide = !t->psFromFront;
          const int32_t *ptex = &sc->sideTex[(pIdx * 2 + pSide) * 3];
          i64 pTop = line_rows(sc, v, g, pIdx, it->viewCeil, x), pBottom = line_rows(sc, v, g, pIdx, it->viewFloor, x);
          i64 pLowerTop = line_rows(sc, v, g, pIdx, pOtherFloor, x), pUpperBottom = line_rows(sc, v, g, pIdx, pOtherCeil, x);
          i64 pct = imax(pTop, c->ceilClip), pcb = imin(pBottom, c->floorClip);
          i64 pcub = imax(imin(pUpperBottom, c->floorClip), pct);
          i64 pclt = imin(imax(pLowerTop, c->ceilClip), pcb);
          int ld = sec_light(sc, it->renderCurrent) != sec_light(sc, pSafeOther);
          int pDrawsUpper = (it->viewCeil > pOtherCeil) && ptex[2] >= 0;
          int pMarksCeil = (it->viewCeil != pOtherCeil) || sec_ctex(sc, it->renderCurrent) != sec_ctex(sc, pSafeOther) || ld;
          if (pDrawsUpper || pMarksCeil) c->ceilClip = pDrawsUpper ? pcub : pct;
          int pDrawsLower = (it->viewFloor < pOtherFloor) && ptex[1] >= 0;
          int pMarksFloor = (it->viewFloor != pOtherFloor) || sec_ftex(sc, it->renderCurrent) != sec_ftex(sc, pSafeOther) || ld;
          if (pDrawsLower || pMarksFloor) c->floorClip = pDrawsLower ? pclt : pcb;
          int pMasked = ptex[0] >= 0;
          int pBottomSil = (it->viewFloor > pOtherFloor) || (v->viewZ < pOtherFloor) || pMasked;
          int pTopSil = (it->viewCeil < pOtherCeil) || (v->viewZ > pOtherCeil) || pMasked;
          for (int y = 0; y < VH; ++y) {
            int in = (pBottomSil && y >= c->floorClip) || (pTopSil && y < c->ceilClip);
            if (in && t->psDist < lb->clip.depth[y * SW + x]) {
              lb->clip.depth[y * SW + x] = t->psDist;
              lb->clip.wall[y * SW + x] = pIdx;
            }
          }
        }
        /* traversal update (engine.py:13242-13371) */
        float prior = c->prev;
        float np = prior;
        if (it->valid) {
          if (t->nokpp) np = t->nopDist;
          else if (t->pskpp) np = t->psDist;
          else if (t->entersShared && (t->osd < it->distance)) np = prior;
          else if (t->usesGeo) np = t->gpDist;
          else np = it->distance;
        }
        if (it->valid && t->epb) np = prior;
        if (it->valid && t->cppb) np = fmaxf(it->distance, c->pendPortalBridgeExit);
        c->prev = np;
        if (t->startsOwner) { c->pendOwnerEp[0] = t->selEp[0]; c->pendOwnerEp[1] = t->selEp[1]; }
        c->pendOwnerBoundary = t->startsOwner || (c->pendOwnerBoundary && t->continuesOwner);
        if (t->endpointOnly) { c->pendEpEp[0] = t->epEp[0]; c->pendEpEp[1] = t->epEp[1]; c->pendEpWall = wallIndex; }
        c->pendEpBoundary = t->endpointOnly;
        if (t->pendEpHasFwd) c->pendEpBridgeIndex = t->epFwdIdx;
        c->pendEpBridgeBoundary = t->pendEpHasFwd;
        int next;
        if (t->nokpp) next = t->nopOther;
        else if (t->pskpp) next = t->psOther;
        else if (t->usesGeo) next = t->gpOther;
        else if (it->valid && !it->oneSided && (t->geometric || t->entersOther || t->entersShared)) next = it->otherSector;
        else if (t->endpointOnly) next = c->cur;
        else next = -1;
        if (t->epb) next = it->otherSector;
        if (t->cppb) next = c->pendPortalBridgeSector;
        if (t->epb) {
          c->pendPortalBridgeIndex = t->ppbIdx;
          c->pendPortalBridgeSector = t->gpOther;
          c->pendPortalBridgeExit = t->gpDist;
        }
        c->pendPortalBridge = t->epb;
        c->cur = next;
      }
    }
    free(trav);
  }
  free(cs);
  free(ci);
}

/* visplane fill (engine.py:13372-13405, 10879-10954, 10588-10616) */
static uint8_t plane_pixel(const Scene *sc, const View *v, int sector, int isFloor, int x, int y) {
  float ph = isFloor ? (v->viewZ - sec_floor(sc, sector)) : (sec_ceil(sc, sector) - v->viewZ);
  int tex = isFloor ? sec_ftex(sc, sector) : sec_ctex(sc, sector);
  const int32_t *ti = &sc->texInfo[tex * 4];
  int wbits = ti[2], hbits = ti[3];
  i64 xscale = 1LL << (32 - wbits), yscale = 1LL << (32 - hbits);
  i64 fs = v->vsin, fc = v->vcos;
  i64 xstep = (xscale * fs) / FOCAL_X, ystep = (yscale * fc) / FOCAL_X;
  i64 col = (i64)x - 159;
  i64 basex = ((xscale * fc) >> 16) + col * xstep;
  i64 basey = ((yscale * -fs) >> 16) + col * ystep;
  i64 pviewx = wrap_mul(xscale, v->vx) >> 16, pviewy = wrap_mul(yscale, -v->vy) >> 16;
  i64 centerRow = v->center >> 16;
  i64 den = (y < centerRow) ? (v->center - (i64)y * FU - FU / 2) : ((i64)y * FU - v->center + FU / 2);
  den = imax(den, 1);
  int overflow = den <= (FOCAL_Y >> 15);
  i64 yslope = (FOCAL_Y << 16) / den;
  if (overflow) yslope = (1LL << 31) - 1;
  i64 phf = rint_f(ph * 65536.0f);
  i64 distance = wrap_mul(phf, yslope) >> 16;
  i64 xfrac = ((wrap_mul(distance, basex) >> 16) + pviewx) & U32MASK;
  i64 yfrac = ((wrap_mul(distance, basey) >> 16) + pviewy) & U32MASK;
  i64 u = xfrac >> (32 - wbits), tv = yfrac >> (32 - hbits);
  uint8_t texel = sc->texAtlas[((size_t)tex * sc->texH + tv) * sc->texW + u];
  i64 light = sec_light(sc, sector) + v->flashLight * 16;
  i64 gv = imin((FLOOR_VIS << 16) / imax(phf, 1), (1LL << 31) - 1);
  i64 rowDist = llabs(v->center - (i64)y * FU);
  i64 vis = imin(wrap_mul(gv, rowDist) >> 16, 24 * FU);
  i64 base = 64 * FU - (light + 12) * (FU / 4);
  int shade = (int)iclamp((base - vis) >> 16, 0, 31);
  return sc->colormap[shade * 256 + texel];
}

/*
 * Per-pixel flat fallback (engine.py:10956-11171): the layer under walls and
 * traversal-marked visplanes.  Every pixel intersects its column ray with each
 * sector's floor / ceiling plane and keeps the nearest hit that lies inside
 * that sector's polygon; unresolved pixels borrow the sector of the next
 * resolved row below (same orientation) and, failing agreement of the nearest
 * anchors left and right, stay with the viewer's sector.
 */
static int sector_at(const Scene *sc, float px, float py);

typedef struct {
  uint8_t resolved[VH * SW];
  int16_t sector[VH * SW];
  float depth[VH * SW];     /* engine.py:11136-11170: ray depth, or the repaired span's plane depth */
} FlatLayer;

static void flat_layer(const Scene *sc, const View *v, int currentSector, FlatLayer *fl) {
  i64 ti = iclamp((ANG90 - v->pitchBam) >> 19, 0, 4095);
  i64 offFixed = ((i64)sc->fineTan[ti] * 12582912LL) >> 16;
  float center = 103.5f + (float)offFixed / 65536.0f;
  uint8_t *unresolved = malloc(VH * SW), *floorPx = malloc(VH * SW), *vspan = malloc(VH * SW), *anchor = malloc(VH * SW);
  for (int x = 0; x < SW; ++x) {
    float rayAngle = v->angle + sc->rayOffsets[x];
    float rc = cosf(rayAngle), rs = sinf(rayAngle);
    float cc = sc->rayCosCorr[x];
    for (int y = 0; y < VH; ++y) {
      float delta = (float)y - center;
      int isFloor = delta > 0;
      float den = fmaxf(fabsf(delta), 0.5f);
      float best = INFINITY;
      int bestSector = currentSector;
      for (int s = 0; s < sc->S; ++s) {
        float ph = isFloor ? (v->viewZ - sc->secF[s * 2]) : (sc->secF[s * 2 + 1] - v->viewZ);
        float perp = ph * 192.0f / den;
        float cd = perp / cc;
        if (!(ph > 0) || !isfinite(cd) || !(cd > 0) || !(cd < best)) continue;
        float px = v->x + rc * cd, py = v->y + rs * cd;
        int crossings = 0;
        for (int k = sc->edgeOff[s]; k < sc->edgeOff[s + 1]; ++k) {
          const float *e = &sc->walls[sc->edgeWalls[k] * 4];
          int crosses = (e[1] > py) != (e[3] > py);
          float dy = e[3] - e[1];
          float safe = fabsf(dy) < 1e-6f ? 1.0f : dy;
          float cx = e[0] + (py - e[1]) * (e[2] - e[0]) / safe;
          crossings += crosses && (px < cx);
        }
        if (crossings & 1) { best = cd; bestSector = s; }
      }
      int i = y * SW + x;
      unresolved[i] = !isfinite(best);
      floorPx[i] = (uint8_t)isFloor;
      fl->sector[i] = (int16_t)bestSector;
      fl->depth[i] = isfinite(best) ? best * cc : INFINITY;
    }
  }
  /* vertical repair: the next resolved row below of the same orientation */
  for (int x = 0; x < SW; ++x) {
    int nextFloor = VH, nextCeil = VH;
    for (int y = VH - 1; y >= 0; --y) {
      int i = y * SW + x;
      if (!unresolved[i] && floorPx[i]) nextFloor = y;
      if (!unresolved[i] && !floorPx[i]) nextCeil = y;
      vspan[i] = 0;
    }
    /* the gathers read the sectors as they were before any repair of this pass;
     * resolved rows are never rewritten, so a bottom-up sweep is equivalent */
    nextFloor = VH; nextCeil = VH;
    for (int y = VH - 1; y >= 0; --y) {
      int i = y * SW + x;
      if (!unresolved[i]) {
        if (floorPx[i]) nextFloor = y; else nextCeil = y;
        continue;
      }
      int next = floorPx[i] ? nextFloor : nextCeil;
      if (next < VH) { fl->sector[i] = fl->sector[next * SW + x]; vspan[i] = 1; }
    }
  }
  /* horizontal repair between the nearest anchors of the row */
  for (int i = 0; i < VH * SW; ++i) anchor[i] = !unresolved[i] || (vspan[i] && fl->sector[i] != currentSector);
  int16_t *repaired = malloc(sizeof(int16_t) * VH * SW);
  memcpy(repaired, fl->sector, sizeof(int16_t) * VH * SW);
  for (int y = 0; y < VH; ++y) {
    int left[SW], right[SW];
    int last = -1;
    for (int x = 0; x < SW; ++x) { if (anchor[y * SW + x]) last = x; left[x] = last; }
    last = SW;
    for (int x = SW - 1; x >= 0; --x) { if (anchor[y * SW + x]) last = x; right[x] = last; }
    for (int x = 0; x < SW; ++x) {
      int i = y * SW + x;
      if (!unresolved[i] || left[x] < 0 || right[x] >= SW) continue;
      int ls = fl->sector[y * SW + left[x]], rs = fl->sector[y * SW + right[x]];
      if (ls == rs) { repaired[i] = (int16_t)ls; vspan[i] = 1; }
    }
  }
  memcpy(fl->sector, repaired, sizeof(int16_t) * VH * SW);
  for (int i = 0; i < VH * SW; ++i) {
    if (!vspan[i]) continue;               /* a vertically or horizontally repaired pixel */
    int y = i / SW, sector = fl->sector[i];
    float ph = floorPx[i] ? (v->viewZ - sc->secF[sector * 2]) : (sc->secF[sector * 2 + 1] - v->viewZ);
    fl->depth[i] = ph * 192.0f / fmaxf(fabsf((float)y - center), 0.5f);
  }
  for (int i = 0; i < VH * SW; ++i) fl->resolved[i] = floorPx[i];  /* reused: 1 = floor pixel */
  free(repaired); free(unresolved); free(floorPx); free(vspan); free(anchor);
}

static float plane_depth(const Scene *sc, const View *v, int sector, int isFloor, int y);

static void plane_pass(const Scene *sc, const View *v, LaneBuffers *lb, int *unownedPixels) {
  int unowned = 0;
  for (int y = 0; y < VH; ++y)
    for (int x = 0; x < SW; ++x) {
      int i = y * SW + x;
      if (lb->filled[i]) continue;
      if (lb->planeSector[i] >= 0) {
        lb->frame[i] = plane_pixel(sc, v, lb->planeSector[i], lb->planeIsFloor[i], x, y);
        lb->sceneDepth[i] = plane_depth(sc, v, lb->planeSector[i], lb->planeIsFloor[i], y);
      } else { lb->frame[i] = 0; lb->sceneDepth[i] = INFINITY; unowned++; }
    }
  if (unowned) {
    /* pixels no seg claimed show the per-pixel fallback layer */
    FlatLayer *fl = malloc(sizeof(FlatLayer));
    flat_layer(sc, v, sector_at(sc, v->x, v->y), fl);
    for (int y = 0; y < VH; ++y)
      for (int x = 0; x < SW; ++x) {
        int i = y * SW + x;
        if (!lb->filled[i] && lb->planeSector[i] < 0) {
          lb->frame[i] = plane_pixel(sc, v, fl->sector[i], fl->resolved[i], x, y);
          lb->sceneDepth[i] = fl->depth[i];
        }
      }
    free(fl);
  }
  if (unownedPixels) *unownedPixels = unowned;
}

/* Two-sided middle textures, replayed after the planes (engine.py:13424-13745):
 * per column the nearest projected crossing of a line that carries a middle
 * texture on the viewer's side, clipped by the drawseg snapshot of the walk. */
static inline i64 trunc_div(i64 a, i64 b) { return a / b; }

static inline i64 masked_iscale(i64 swall) {
  i64 s = (swall * FU) >> 18;
  if (s >= 0 && s < 3) return 3;
  if (s > -3 && s < 0) return -3;
  return s;
}

static void masked_pass(const Scene *sc, const View *v, const LaneGeom *g, LaneBuffers *lb) {
  const int W = sc->W;
  for (int x = 0; x < SW; ++x) {
    float best = INFINITY;
    int w = -1, side = 0, texId = -1;
    for (int k = 0; k < W; ++k) {
      if (sc->wsec[k * 2 + 1] < 0) continue;
      int sd = g->wv[k].frontFacingF ? 0 : 1;
      int t = sc->sideTex[(k * 2 + sd) * 3];
      if (t < 0 || !g->proj[(size_t)x * W + k]) continue;
      float d = g->dist[(size_t)x * W + k];
      if (d < best) { best = d; w = k; side = sd; texId = t; }
    }
    if (!isfinite(best)) continue;
    const WallView *wv = &g->wv[w];
    int front = sc->wsec[w * 2], back = sc->wsec[w * 2 + 1] < 0 ? 0 : sc->wsec[w * 2 + 1];
    int lightSector = side == 0 ? front : back;
    float worldTop = fminf(sec_ceil(sc, front), sec_ceil(sc, back));
    const int32_t *ti = &sc->texInfo[texId * 4];
    int tw = ti[0], th = ti[1], hbits = ti[3];
    i64 owallTop = line_rows(sc, v, g, w, worldTop, x);
    i64 owallBottom = line_rows(sc, v, g, w, worldTop - (float)th, x);
    int hasSaved = lb->maskedWall[x] == w;
    i64 ceilClip = imax(owallTop, hasSaved ? lb->maskedCeil[x] : 0);
    i64 floorClip = imin(owallBottom, hasSaved ? lb->maskedFloor[x] : VH);
    const float *soff = &sc->sideOff[(w * 2 + side) * 2];
    i64 hoff, vstepBase;
    prep_wall(sc, wv, w, x, &hoff, &vstepBase);
    i64 repeat = rint_f(sc->wlen[w] * 65536.0f);
    if (side != 0) hoff = repeat - hoff;
    if (wv->sl > 0 && hoff < 0) hoff = 0;
    if (hoff >= repeat) hoff = repeat - 1;
    i64 u = pymod((hoff + rint_f(soff[0] * 65536.0f)) >> 16, tw);
    i64 vstep = vstepBase * (1LL << (14 - hbits));
    i64 texMid = rint_f((worldTop - v->viewZ) * 65536.0f + soff[1] * 65536.0f);
    /* R_DrawMaskedColumn: post rows from the drawseg's interpolated scale */
    i64 sLeft = iclamp(wv->sl, 0, SW - 1), sLast = iclamp(wv->sr - 1, 0, SW - 1);
    i64 dummy, startSwall, endSwall;
    prep_wall(sc, wv, w, (int)sLeft, &dummy, &startSwall);
    prep_wall(sc, wv, w, (int)sLast, &dummy, &endSwall);
    i64 startScale = trunc_div(1LL << 32, masked_iscale(startSwall));
    i64 endScale = trunc_div(1LL << 32, masked_iscale(endSwall));
    i64 span = imax(wv->sr - wv->sl, 1);
    i64 scaleStep = trunc_div(endScale - startScale, span);
    i64 spriteScale = startScale + wrap_mul(scaleStep, (i64)x - wv->sl);
    i64 topScreen = v->center - (wrap_mul(texMid, spriteScale) >> 16);
    i64 postTop = topScreen >> 16;
    i64 postBottom = ((topScreen + wrap_mul(spriteScale, th) - FU) >> 16) + 1;
    i64 clippedTop = imax(postTop, ceilClip), clippedBottom = imin(postBottom, floorClip);
    i64 dcIscale = (vstepBase * FU) >> 18;
    int initialPost = clippedTop < clippedBottom;
    i64 fracStart = texMid + wrap_mul(clippedTop, dcIscale) - (wrap_mul(v->center - FU, dcIscale) >> 16);
    i64 fracEnd = fracStart + wrap_mul(clippedBottom - clippedTop - 1, dcIscale);
    if (initialPost && clippedBottom < floorClip && fracEnd < (i64)th * FU - dcIscale) clippedBottom += 1;
    if (!(hasSaved || g->left[(size_t)x * W + w])) continue;
    const float *wl = &sc->walls[w * 4];
    int horizontal = fabsf(wl[3] - wl[1]) < 1e-6f, vertical = fabsf(wl[2] - wl[0]) < 1e-6f;
    i64 light = sec_light(sc, lightSector) + v->flashLight * 16 + (vertical ? 16 : (horizontal ? -16 : 0));
    i64 vis = line_vis(sc, g, w, side, x);
    int shade = wall_shade(light, vis);
    for (i64 y = imax(clippedTop, 0); y < imin(clippedBottom, VH); ++y) {
      i64 screenDelta = y * FU - v->center + FU;
      i64 frac = shl(texMid, 16 - hbits) + (wrap_mul(vstep, screenDelta) >> 16);
      i64 tv = (frac & U32MASK) >> (32 - hbits);
      uint8_t texel = sc->texAtlas[((size_t)texId * sc->texH + tv) * sc->texW + u];
      lb->frame[y * SW + x] = sc->colormap[shade * 256 + texel];
      lb->sceneDepth[y * SW + x] = best;
    }
  }
}

/* point-in-sector for actors (engine.py:9598-9617) */
static int sector_at(const Scene *sc, float px, float py) {
  for (int s = 0; s < sc->S; ++s) {
    int crossings = 0;
    for (int k = sc->edgeOff[s]; k < sc->edgeOff[s + 1]; ++k) {
      const float *e = &sc->walls[sc->edgeWalls[k] * 4];
      float x1 = e[0], y1 = e[1], x2 = e[2], y2 = e[3];
      int crosses = (y1 > py) != (y2 > py);
      float dy = y2 - y1;
      float safe = fabsf(dy) < 1e-6f ? 1.0f : dy;
      float cx = x1 + (py - y1) * (x2 - x1) / safe;
      crossings += crosses && (px < cx);
    }
    if (crossings & 1) return s;
  }
  return 0;
}

static float wrap_angle(float a) {
  /* torch.remainder(a + pi, 2*pi) - pi in float32 */
  const float pi = (float)M_PI, twoPi = (float)(2 * M_PI);
  float t = a + pi;
  float r = fmodf(t, twoPi);
  if (r != 0 && ((r < 0) != (twoPi < 0))) r += twoPi;
  return r - pi;
}

/*
 * The per-pixel flat fallback (engine.py:10961-11026) leaves a pixel unresolved
 * when the hit of its column ray with no sector's floor / ceiling plane lies
 * inside that sector's polygon.  Only that yes/no leaks into the final frame:
 * a visplane pixel that is unresolved clips sprites at its plane depth
 * (engine.py:13406-13422).
 */
static int pixel_unresolved(const Scene *sc, const View *v, int x, int y) {
  i64 ti = iclamp((ANG90 - v->pitchBam) >> 19, 0, 4095);
  i64 offFixed = ((i64)sc->fineTan[ti] * 12582912LL) >> 16;
  float pitchOff = (float)offFixed / 65536.0f;
  float center = 103.5f + pitchOff;
  float rayAngle = v->angle + sc->rayOffsets[x];
  float rc = cosf(rayAngle), rs = sinf(rayAngle);
  float cc = sc->rayCosCorr[x];
  float delta = (float)y - center;
  int floorPixel = delta > 0;
  float den = fmaxf(fabsf(delta), 0.5f);
  for (int s = 0; s < sc->S; ++s) {
    float ph = floorPixel ? (v->viewZ - sc->secF[s * 2]) : (sc->secF[s * 2 + 1] - v->viewZ);
    float perp = ph * 192.0f / den;
    float cd = perp / cc;
    if (!(ph > 0) || !isfinite(cd) || !(cd > 0)) continue;
    float px = v->x + rc * cd, py = v->y + rs * cd;
    int crossings = 0;
    for (int k = sc->edgeOff[s]; k < sc->edgeOff[s + 1]; ++k) {
      const float *e = &sc->walls[sc->edgeWalls[k] * 4];
      float x1 = e[0], y1 = e[1], x2 = e[2], y2 = e[3];
      int crosses = (y1 > py) != (y2 > py);
      float dy = y2 - y1;
      float safe = fabsf(dy) < 1e-6f ? 1.0f : dy;
      float cx = x1 + (py - y1) * (x2 - x1) / safe;
      crossings += crosses && (px < cx);
    }
    if (crossings & 1) return 0;
  }
  return 1;
}

static float plane_depth(const Scene *sc, const View *v, int sector, int isFloor, int y) {
  i64 ti = iclamp((ANG90 - v->pitchBam) >> 19, 0, 4095);
  i64 offFixed = ((i64)sc->fineTan[ti] * 12582912LL) >> 16;
  float pitchOff = (float)offFixed / 65536.0f;
  float flatCenter = (103.0f + pitchOff) + 0.5f;
  float ph = isFloor ? (v->viewZ - sec_floor(sc, sector)) : (sec_ceil(sc, sector) - v->viewZ);
  float den = fmaxf(fabsf((float)y - flatCenter), 0.5f);
  return ph * 192.0f / den;
}


/* ---- bullet-chip decals (engine.py:13747-13991) --------------------------------
 * The chips of a lane, oldest first, are shaded onto the wall pixels whose surface
 * depth equals the chip's own ray depth.  `decals` is the lane's ring of `slots`
 * records; a slot with serial < 0 is free. */
static void decal_pass(const Scene *sc, const View *v, const LaneGeom *g, LaneBuffers *lb, const gd_decal *decals,
                       int slots) {
  if (!decals || slots <= 0 || sc->decals <= 0) return;
  int *order = malloc(sizeof(int) * (size_t)slots);
  int n = 0;
  for (int s = 0; s < slots; ++s)
    if (decals[s].serial >= 0) order[n++] = s;
  /* ascending serial (engine.py:13763-13775); serials of a lane are distinct */
  for (int i = 1; i < n; ++i) {
    int s = order[i], j = i - 1;
    while (j >= 0 && decals[order[j]].serial > decals[s].serial) { order[j + 1] = order[j]; --j; }
    order[j + 1] = s;
  }
  const i64 ti = iclamp((ANG90 - v->pitchBam) >> 19, 0, 4095);
  const i64 offFixed = ((i64)sc->fineTan[ti] * 12582912LL) >> 16;   /* round(192 * 65536) */
  const float center = 104.0f + (float)offFixed / 65536.0f;        /* engine.py:13785-13789 */
  const float width = (float)sc->decalW;
  for (int k = 0; k < n; ++k) {
    const gd_decal *d = &decals[order[k]];
    int w = (int)iclamp(d->wall, 0, sc->W - 1);
    int style = d->style;
    int variant = style % 5, flipX = (style / 5) % 2, flipY = (style / 10) % 2, side = style / 20;
    if (variant >= sc->decals || side > 1) continue;   /* the engine writes sides 0 and 1 only (engine.py:6280-6306) */
    const float *wl = &sc->walls[w * 4];
    float vecx = wl[2] - wl[0], vecy = wl[3] - wl[1];
    float impx = wl[0] + d->along * vecx, impy = wl[1] + d->along * vecy;
    /* tangent: the fine-angle direction of the wall as seen from the chip's side */
    int fine = sc->wallFine[w * 2 + side] & 8191;
    float tanx = (float)sc->fineSine[(fine + 2048) & 8191] / 65536.0f, tany = (float)sc->fineSine[fine] / 65536.0f;
    float leftOff = (float)sc->decalInfo[variant * 4 + 1], topOff = (float)sc->decalInfo[variant * 4 + 2];
    int height = sc->decalInfo[variant * 4 + 0];
    float a = leftOff * GD_DECAL_SCALE, b = (width - leftOff) * GD_DECAL_SCALE;
    float lx = impx - tanx * a, ly = impy - tany * a;
    float rx_ = impx + tanx * b, ry_ = impy + tany * b;
    float segx = rx_ - lx, segy = ry_ - ly;
    /* FWallCoords on the chip's two fixed-point endpoints (engine.py:13837-13883) */
    i64 ex[2] = {rint_f(lx * 65536.0f), rint_f(rx_ * 65536.0f)}, ey[2] = {rint_f(ly * 65536.0f), rint_f(ry_ * 65536.0f)};
    i64 tx[2], ty[2];
    for (int e = 0; e < 2; ++e) {
      i64 relx = ex[e] - v->vx, rely = ey[e] - v->vy;
      tx[e] = (relx * v->vsin - rely * v->vcos) >> 20;
      ty[e] = (relx * v->vcos + rely * v->vsin) >> 20;
    }
    const i64 cf = 160 * FU;
    i64 sty1 = ty[0] == 0 ? 1 : ty[0], sty2 = ty[1] == 0 ? 1 : ty[1];
    i64 pl = ((cf + (tx[0] * cf) / sty1) >> 16) + (tx[0] >= 0);
    i64 pr = ((cf + (tx[1] * cf) / sty2) >> 16) + (tx[1] >= 0);
    i64 lden = tx[0] - tx[1] - ty[1] + ty[0], rden = ty[1] - ty[0] - tx[1] + tx[0];
    int leftInside = tx[0] >= -ty[0] && tx[0] <= ty[0] && ty[0] != 0;
    int rightInside = tx[1] <= ty[1] && tx[1] >= -ty[1] && ty[1] != 0;
    int leftClipped = tx[0] < -ty[0] && tx[1] >= -ty[1] && lden != 0;
    int rightClipped = tx[1] > ty[1] && tx[0] <= ty[0] && rden != 0;
    i64 screenL = leftInside ? iclamp(pl, 0, SW) : 0, screenR = rightInside ? iclamp(pr, 0, SW) : SW;
    if (!((leftInside || leftClipped) && (rightInside || rightClipped) && screenR > screenL)) continue;
    float cross = vecx * (v->y - wl[1]) - vecy * (v->x - wl[0]);
    if ((cross > 0 ? 1 : 0) != side) continue;
    int sector = sc->wsec[w * 2 + side];
    if (sector < 0) sector = 0;
    int horizontal = fabsf(vecy) < 1e-6f, vertical = fabsf(vecx) < 1e-6f;
    i64 light = (i64)sec_light(sc, sector) + (vertical ? 16 : (horizontal ? -16 : 0)) + v->flashLight * 16;
    float offx = lx - v->x, offy = ly - v->y;
    for (int x = (int)screenL; x < (int)screenR; ++x) {
      float rx = g->dirx[x], ry = g->diry[x];
      float den = rx * segy - ry * segx;
      if (fabsf(den) < 1e-6f) continue;
      float distance = (offx * segy - offy * segx) / den;
      float along = (offx * ry - offy * rx) / den;
      if (!(distance > 0)) continue;
      i64 u = (i64)floorf(along * width);
      u = iclamp(u, 0, sc->decalW - 1);
      if (flipX) u = sc->decalW - 1 - u;
      float safeDist = fmaxf(distance, 1e-6f);
      float vscale = 96.0f / safeDist;
      float top = center - ((d->z + topOff * GD_DECAL_SCALE) - v->viewZ) * 192.0f / safeDist;
      i64 depthFixed = rint_f(safeDist * 4096.0f);
      i64 vis = (WALL_VIS << 12) / imax(depthFixed, 1);
      int shade = wall_shade(light, vis);
      for (int y = 0; y < VH; ++y) {
        i64 tv = (i64)floorf(((float)y - top) / vscale);
        if (tv < 0 || tv >= height) continue;
        if (flipY) tv = height - 1 - tv;
        uint8_t src = sc->decalAtlas[((size_t)variant * sc->decalH + tv) * sc->decalW + u];
        if (!src) continue;
        int i = y * SW + x;
        if (!(fabsf(lb->sceneDepth[i] - distance) <= 1e-3f)) continue;
        uint8_t opacity = sc->decalOpacity[shade * 256 + src];
        lb->frame[i] = sc->decalBlack[opacity * 256 + lb->frame[i]];
      }
    }
  }
  free(order);
}

/* per calling thread: the tests render chunks of lanes from several threads at once */
static __thread const gd_decal *gBoundDecals;
static __thread int gBoundDecalSlots;
/* Decal rings of the lanes of the next gd_oracle_render calls: n x slots records, or NULL. */
void gd_oracle_bind_decals(const gd_decal *decals, int slots) {
  gBoundDecals = decals;
  gBoundDecalSlots = slots;
}

typedef struct {
  int alive;
  float x, y, z, depth;
  i64 depthFixed;
  i64 left, right, xstep, yscale, topFixed, texMid, iscale;
  int sprite, w, h, bright, style, light;
} Actor;

static void sprite_pass(const Scene *sc, const View *v, const LaneGeom *g, LaneBuffers *lb,
                        const gd_thing *things, int nThings, const float *depthOverride) {
  if (nThings <= 0) return;
  Actor *A = calloc((size_t)nThings, sizeof(Actor));
  int *order = malloc(sizeof(int) * (size_t)nThings);
  for (int a = 0; a < nThings; ++a) {
    const gd_thing *t = &things[a];
    Actor *ac = &A[a];
    ac->alive = (t->flags & GD_THING_ALIVE) != 0;
    ac->bright = (t->flags & GD_THING_BRIGHT) != 0;
    ac->style = t->style;
    ac->x = t->x; ac->y = t->y; ac->z = t->z;
    ac->sprite = t->sprite;
    const int32_t *si = &sc->sprInfo[ac->sprite * 4];
    ac->w = si[0]; ac->h = si[1];
    float dx = ac->x - v->x, dy = ac->y - v->y;
    float dist = sqrtf(dx * dx + dy * dy);
    if (dist < 1.0f) dist = 1.0f;
    float rel = wrap_angle(atan2f(dy, dx) - v->angle);
    ac->depth = depthOverride ? depthOverride[a] : dist * cosf(rel);
    i64 ax = rint_f(ac->x * 65536.0f), ay = rint_f(ac->y * 65536.0f);
    i64 rx = ax - v->vx, ry = ay - v->vy;
    i64 depthFixed = (rx * v->vcos + ry * v->vsin) >> 20;
    i64 sideFixed = (rx * v->vsin - ry * v->vcos) >> 16;
    ac->depthFixed = depthFixed;
    i64 xscale = (FOCAL_X << 12) / imax(depthFixed, SPRITE_MIN_DEPTH);
    i64 leftFixed = sideFixed - (i64)si[2] * FU;
    ac->left = 160 + (wrap_mul(leftFixed, xscale) >> 32);
    i64 rightFixed = leftFixed + (i64)si[0] * FU;
    ac->right = 160 + (wrap_mul(rightFixed, xscale) >> 32);
    ac->xstep = ((i64)si[0] << 16) / imax(ac->right - ac->left, 1);
    ac->yscale = (FOCAL_Y << 12) / imax(depthFixed, SPRITE_MIN_DEPTH);
    ac->texMid = (i64)si[3] * FU - rint_f((v->viewZ - ac->z) * 65536.0f);
    ac->topFixed = v->center - (wrap_mul(ac->texMid, ac->yscale) >> 16);
    ac->iscale = U32MASK / imax(ac->yscale, 1);
    ac->light = sec_light(sc, sector_at(sc, ac->x, ac->y));
  }
  for (int x = 0; x < SW; ++x) {
    int n = 0;
    int bw = g->blockingWall[x];
    const WallView *bwv = &g->wv[bw];
    i64 bnear = imin(bwv->dl, bwv->dr), bfar = imax(bwv->dl, bwv->dr);
    const float *bg = &sc->walls[bw * 4];
    float bdx = bg[2] - bg[0], bdy = bg[3] - bg[1];
    int bowns = x >= bwv->sl && x < bwv->sr;
    for (int a = 0; a < nThings; ++a) {
      const Actor *ac = &A[a];
      if (!(ac->alive && x >= ac->left && x < ac->right && ac->depth > 0)) continue;
      int rayVisible = ac->depth < g->wallDistance[x];
      float bside = bdx * (ac->y - bg[1]) - bdy * (ac->x - bg[0]);
      int behind = (bnear > ac->depthFixed) || ((bfar > ac->depthFixed) && (bside <= 0));
      rayVisible |= !bowns || behind;
      if (rayVisible) order[n++] = a;
    }
    /* stable insertion sort by depth ascending, then paint far to near */
    for (int i = 1; i < n; ++i) {
      int a = order[i], j = i - 1;
      while (j >= 0 && A[order[j]].depth > A[a].depth) { order[j + 1] = order[j]; --j; }
      order[j + 1] = a;
    }
    for (int k = n - 1; k >= 0; --k) {
      const Actor *ac = &A[order[k]];
      i64 u = (((i64)x - ac->left) * ac->xstep) >> 16;
      if (u < 0 || u >= ac->w) continue;
      i64 light = ac->light + v->flashLight * 16;
      if (ac->bright) light = 255;
      float base = 61.0f - (float)light / 4.0f;
      float visf = fminf(1280.0f / fmaxf(ac->depth, 1.0f), 24.0f);
      int shade = (int)iclamp((i64)floorf(base - visf), 0, 31);
      for (int y = 0; y < VH; ++y) {
        i64 frac = ac->texMid + (i64)y * ac->iscale - (wrap_mul(v->center - FU, ac->iscale) >> 16);
        i64 tv = frac >> 16;
        if (tv < 0 || tv >= ac->h) continue;
        int i = y * SW + x;
        int cw = lb->clip.wall[i];
        int visible;
        if (cw >= 0) {
          const WallView *cwv = &g->wv[cw];
          i64 cnear = imin(cwv->dl, cwv->dr), cfar = imax(cwv->dl, cwv->dr);
          const float *cg = &sc->walls[cw * 4];
          float cdx = cg[2] - cg[0], cdy = cg[3] - cg[1];
          float cside = cdx * (ac->y - cg[1]) - cdy * (ac->x - cg[0]);
          visible = (cnear > ac->depthFixed) || ((cfar > ac->depthFixed) && (cside <= 0));
        } else {
          float limit = lb->clip.depth[i];
          if (isinf(limit) && !lb->filled[i] && lb->planeSector[i] >= 0 && pixel_unresolved(sc, v, x, y))
            limit = plane_depth(sc, v, lb->planeSector[i], lb->planeIsFloor[i], y);
          visible = ac->depth < limit;
        }
        if (!visible) continue;
        size_t si = ((size_t)ac->sprite * sc->sprH + (size_t)tv) * sc->sprW + (size_t)u;
        uint8_t post = sc->sprPost[si];
        if (post == 255) continue;
        i64 postTop = (ac->topFixed + ac->yscale * (i64)post) >> 16;
        if (y < postTop) continue;
        uint8_t lit = sc->colormap[shade * 256 + sc->sprAtlas[si]];
        uint8_t dst = lb->frame[i];
        uint8_t out = lit;
        if (ac->style == -2) out = sc->transLut[dst * 256 + lit];
        else if (ac->style >= 0) out = sc->addLut[((ac->style > 1 ? 1 : ac->style) * 256 + dst) * 256 + lit];
        lb->frame[i] = out;
      }
    }
  }
  free(A);
  free(order);
}

/* psprite composite (engine.py:14994-15121) */
static void weapon_patch(const Scene *sc, uint8_t *frame, int id, i64 hoff, i64 voff) {
  const int32_t *wi = &sc->wpnInfo[id * 4];
  i64 w = wi[0], h = wi[1], left = wi[2], top = wi[3];
  i64 screenLeft = (hoff - left * FU) >> 16;
  i64 texMid = 100 * FU - (32 * FU + 0x6000) - voff + top * FU;
  i64 yscale = GD_SCREEN_H * FU / 200;
  i64 iscale = U32MASK / yscale;
  for (int y = 0; y < VH; ++y) {
    i64 sy = (texMid + ((i64)y - (VH / 2 - 1)) * iscale) >> 16;
    if (sy < 0 || sy >= h) continue;
    i64 cy = iclamp(sy, 0, sc->wpnH - 1);
    for (int x = 0; x < SW; ++x) {
      i64 sx = (i64)x - screenLeft;
      if (sx < 0 || sx >= w) continue;
      i64 cx = iclamp(sx, 0, sc->wpnW - 1);
      size_t si = ((size_t)id * sc->wpnH + (size_t)cy) * sc->wpnW + (size_t)cx;
      if (sc->wpnOpaque[si]) frame[y * SW + x] = sc->wpnAtlas[si];
    }
  }
}

static void weapon_pass(const Scene *sc, const int32_t *lane, uint8_t *frame) {
  if (!sc->wpnAvailable) return;
  int weapon = (int)iclamp(lane[GD_L_WEAPON], 0, 7);
  int cooldown = (int)iclamp(lane[GD_L_WPN_COOLDOWN], 0, sc->wpnTics - 1);
  int parity = (int)pymod(lane[GD_L_WPN_FIRE_COUNT], 2);
  if (weapon == 1 && cooldown == 0) parity = (int)pymod(imax(lane[GD_L_WPN_READY_TICS] - 1, 0) / 4, 2);
  int ti = (weapon * 2 + parity) * sc->wpnTics + cooldown;
  int frameId = sc->wpnFrameIds[ti], flashId = sc->wpnFlashIds[ti];
  i64 lowerTics = iclamp(16 - lane[GD_L_WPN_LOWER], 0, 16);
  i64 verticalTics = lane[GD_L_WPN_PENDING] >= 0 ? lowerTics : lane[GD_L_WPN_RAISE];
  i64 spawnRaise = iclamp(14 - ((i64)lane[GD_L_EPISODE_TIME] - 1), 0, 14);
  verticalTics = imax(verticalTics, spawnRaise);
  int ready = lane[GD_L_WPN_COOLDOWN] <= 0 && lane[GD_L_WPN_RAISE] <= 0 && lane[GD_L_WPN_PENDING] < 0;
  i64 bobAngle = ((i64)lane[GD_L_EPISODE_TIME] * 128) & 8191;
  i64 bob = lane[GD_L_BOB_FIXED];
  i64 bobx = (bob * sc->fineSine[(bobAngle + 2048) & 8191]) >> 16;
  i64 boby = (bob * sc->fineSine[bobAngle & 4095]) >> 16;
  if (!ready) { bobx = 0; boby = 0; }
  int visible = !(lane[GD_L_FLAGS] & 1);
  if (!visible) return;
  i64 voff = verticalTics * 6 * FU + boby;
  weapon_patch(sc, frame, frameId, bobx, voff);
  if (flashId >= 0) weapon_patch(sc, frame, flashId, bobx, voff);
}

/* status bar (engine.py:15158-15267) */
static void hud_patch(const Scene *sc, uint8_t *canvas, int patch, int x, int y) {
  const int32_t *hi = &sc->hudInfo[patch * 4];
  x -= hi[2];
  y -= hi[3];
  int w = hi[0], h = hi[1];
  if (w <= 0 || h <= 0) return;
  int sx = x < 0 ? -x : 0, sy = y < 0 ? -y : 0;
  int tx = x > 0 ? x : 0, ty = y > 0 ? y : 0;
  int cw = (w - sx) < (SW - tx) ? (w - sx) : (SW - tx);
  int ch = (h - sy) < (GD_HUD_H - ty) ? (h - sy) : (GD_HUD_H - ty);
  if (cw <= 0 || ch <= 0) return;
  for (int j = 0; j < ch; ++j)
    for (int i = 0; i < cw; ++i) {
      size_t si = ((size_t)patch * GD_HUD_H + (size_t)(sy + j)) * SW + (size_t)(sx + i);
      if (sc->hudOpaque[si]) canvas[(ty + j) * SW + tx + i] = sc->hudAtlas[si];
    }
}

static void hud_number(const Scene *sc, uint8_t *canvas, int value, int right, int y, int small) {
  int vclamped = value < -99 ? -99 : (value > 999 ? 999 : value);
  char text[8];
  int len = 0;
  {
    int neg = vclamped < 0;
    int mag = neg ? -vclamped : vclamped;
    char tmp[8];
    int n = 0;
    do { tmp[n++] = (char)('0' + mag % 10); mag /= 10; } while (mag > 0);
    if (neg) text[len++] = '-';
    while (n > 0) text[len++] = tmp[--n];
  }
  int dw = small ? 4 : 14, base = small ? 28 : 2;
  int x = right - len * dw;
  for (int k = 0; k < len; ++k) {
    if (text[k] != '-') {
      int patch = base + (text[k] - '0');
      const int32_t *hi = &sc->hudInfo[patch * 4];
      hud_patch(sc, canvas, patch, x - hi[2], y - hi[3]);
    }
    x += dw;
  }
}

static const int WEAPON_AMMO_SLOT[8] = {-1, -1, 1, 2, 2, 1, 4, 5};

static void hud_pass(const Scene *sc, const int32_t *lane, uint8_t *canvas) {
  const float *lf = (const float *)lane;
  memset(canvas, 0, (size_t)GD_HUD_H * SW);
  hud_patch(sc, canvas, 0, 0, 0);
  hud_patch(sc, canvas, 1, 104, 0);
  int weapon = lane[GD_L_WEAPON];
  int ammoSlot = WEAPON_AMMO_SLOT[weapon < 0 ? 0 : (weapon > 7 ? 7 : weapon)];
  int ammo = ammoSlot < 0 ? 0 : (int)lf[GD_L_READY_AMMO];
  float hf = lf[GD_L_HEALTH], af = lf[GD_L_ARMOR];
  int health = (int)(hf < 0 ? 0 : (hf > 999 ? 999 : hf));
  int armor = (int)(af < 0 ? 0 : (af > 999 ? 999 : af));
  hud_number(sc, canvas, ammo, 44, 3, 0);
  hud_number(sc, canvas, health, 90, 3, 0);
  hud_patch(sc, canvas, 12, 90, 3);
  hud_number(sc, canvas, armor, 221, 3, 0);
  hud_patch(sc, canvas, 12, 221, 3);
  int pain = (100 - health) / 20;  /* python floor division on non-negative operand below */
  if (100 - health < 0) pain = -((health - 100 + 19) / 20);
  pain = pain < 0 ? 0 : (pain > 4 ? 4 : pain);
  int face = 13 + pain * 3 + lane[GD_L_FACE_INDEX];
  if (lane[GD_L_GRIN_TICS] > 0) face = 64 + pain;
  else if (lane[GD_L_PAIN_TICS] > 0) {
    if (lane[GD_L_FLAGS] & 2) face = 59 + pain;
    else {
      static const int dirBase[3] = {44, 49, 54};
      int d = lane[GD_L_PAIN_DIRECTION];
      face = dirBase[d < 0 ? 0 : (d > 2 ? 2 : d)] + pain;
    }
  } else if (lane[GD_L_ATTACK_HELD] >= 70) face = 49 + pain;
  if (health <= 0) face = 69;
  hud_patch(sc, canvas, face, 143, 0);
  static const int armsXY[6][2] = {{111, 4}, {123, 4}, {135, 4}, {111, 14}, {123, 14}, {135, 14}};
  for (int wi = 0; wi < 6; ++wi) {
    int owned = wi < 5 && ((lane[GD_L_WEAPONS_OWNED] >> (wi + 1)) & 1);
    int patch = owned ? 28 + wi + 2 : 38 + wi;
    hud_patch(sc, canvas, patch, armsXY[wi][0], armsXY[wi][1]);
  }
  static const int maxima[4] = {200, 50, 50, 300};
  for (int row = 0; row < 4; ++row) {
    int y = 5 + row * 6;
    hud_number(sc, canvas, (int)lf[GD_L_AMMO0 + row], 288, y, 1);
    hud_number(sc, canvas, maxima[row], 314, y, 1);
  }
}

/* integer 320x240 -> 84x84 area resize and grayscale
 * (src/gradoom/_triton_kernels.py:120-177).  Rows >= srcRows read as black. */
/* PLAYPAL of one lane: the plain palette, or its bonus / damage blends when the
 * lane asks for screen flashes (engine.py:15381-15398; float32, separately
 * rounded operations, truncating conversion). */
static void lane_palette(const Scene *sc, const int32_t *lane, uint8_t *pal) {
  memcpy(pal, sc->playpal, 768);
  int flags = lane ? lane[GD_L_FLAGS] : 0;
  if (!(flags & 4)) return;
  int damage = (flags >> 8) & 0xFF, bonusCount = (flags >> 16) & 0xFF;
  if (damage > 113) damage = 113;
  float bonus = fminf((float)bonusCount * 8.0f, 128.0f) / 255.0f;
  float flash = sc->damageAlpha[damage] / 255.0f;
  static const float gold[3] = {215.0f, 186.0f, 69.0f}, red[3] = {255.0f, 0.0f, 0.0f};
  for (int i = 0; i < 256; ++i)
    for (int c = 0; c < 3; ++c) {
      float a = (float)sc->playpal[i * 3 + c] * (1.0f - bonus);
      float b = gold[c] * bonus;
      float rgb = a + b;
      float d = rgb * (1.0f - flash);
      float e = red[c] * flash;
      float out = d + e;
      out = out < 0.0f ? 0.0f : (out > 255.0f ? 255.0f : out);
      pal[i * 3 + c] = (uint8_t)out;
    }
}

static void area_resize(const uint8_t *playpal, const uint8_t *indexed, int srcRows, uint8_t *out) {
  for (int oy = 0; oy < GD_OBS; ++oy)
    for (int ox = 0; ox < GD_OBS; ++ox) {
      int ys = oy * 240, ye = (oy + 1) * 240, xs = ox * 320, xe = (ox + 1) * 320;
      i64 sum[3] = {0, 0, 0};
      for (int sy = ys / 84; sy < 240 && sy * 84 < ye; ++sy) {
        int yo = (ye < (sy + 1) * 84 ? ye : (sy + 1) * 84) - (ys > sy * 84 ? ys : sy * 84);
        if (yo <= 0) continue;
        for (int sx = xs / 84; sx < 320 && sx * 84 < xe; ++sx) {
          int xo = (xe < (sx + 1) * 84 ? xe : (sx + 1) * 84) - (xs > sx * 84 ? xs : sx * 84);
          if (xo <= 0) continue;
          int wgt = (yo * xo) / 48;
          if (sy >= srcRows) continue;
          const uint8_t *rgb = &playpal[indexed[sy * SW + sx] * 3];
          sum[0] += rgb[0] * wgt; sum[1] += rgb[1] * wgt; sum[2] += rgb[2] * wgt;
        }
      }
      i64 r = (sum[0] + 800) / 1600, gch = (sum[1] + 800) / 1600, b = (sum[2] + 800) / 1600;
      out[oy * GD_OBS + ox] = (uint8_t)((r * 77 + gch * 150 + b * 29 + 128) >> 8);
    }
}

/* ---- public entry points (called through ctypes by the tests) ----------- */

typedef struct {
  Scene sc;
  LaneGeom g;
  LaneBuffers *lb;
} Ctx;

static Ctx *ctx_new(const uint8_t *blob) {
  Ctx *c = calloc(1, sizeof(Ctx));
  if (scene_open(&c->sc, blob) != 0) { free(c); return NULL; }
  int W = c->sc.W;
  c->g.wv = calloc((size_t)W, sizeof(WallView));
  c->g.dist = malloc(sizeof(float) * SW * (size_t)W);
  c->g.along = malloc(sizeof(float) * SW * (size_t)W);
  c->g.geo = malloc((size_t)SW * W);
  c->g.proj = malloc((size_t)SW * W);
  c->g.left = malloc((size_t)SW * W);
  c->g.eoIdx = malloc(sizeof(int32_t) * SW * (size_t)W);
  c->g.eoDist = malloc(sizeof(float) * SW * (size_t)W);
  c->g.frag = calloc((size_t)(c->sc.F > 0 ? c->sc.F : 1), sizeof(WallView));
  c->lb = malloc(sizeof(LaneBuffers));
  return c;
}
static void ctx_free(Ctx *c) {
  free(c->g.frag); free(c->g.wv); free(c->g.dist); free(c->g.along); free(c->g.geo); free(c->g.proj); free(c->g.left);
  free(c->g.eoIdx); free(c->g.eoDist); free(c->lb); free(c);
}

/*
 * Render `n` lanes.  Outputs (any may be NULL):
 *   indexed  n x 240 x 320 u8   view + status bar, palette indices
 *   obs      n x 84 x 84 u8     grayscale observation (status bar masked when mask_hud)
 *   stages   n x 3 x 208 x 320 u8  frame after walls+planes, after sprites, after weapon
 *   unowned  n i32              pixels neither wall nor marked plane
 * things: n x max_things records; depth_override: optional n x max_things f32.
 * stage_mask bit0 walls/planes, bit1 sprites, bit2 weapon, bit3 hud.
 */
int gd_oracle_render(const uint8_t *blob, const int32_t *lanes, const gd_thing *things, int max_things,
                     const float *depth_override, int n, int mask_hud, int stage_mask, uint8_t *indexed,
                     uint8_t *obs, uint8_t *stages, int32_t *unowned) {
  Ctx *c = ctx_new(blob);
  if (!c) return -1;
  uint8_t *full = malloc((size_t)GD_SCREEN_H * SW);
  for (int l = 0; l < n; ++l) {
    const int32_t *lane = &lanes[(size_t)l * GD_LANE_WORDS];
    View v;
    view_setup(&c->sc, lane, &v);
    lane_geometry(&c->sc, &v, &c->g);
    memset(c->lb->frame, 0, sizeof c->lb->frame);
    int un = 0;
    if (stage_mask & 1) {
      wall_pass(&c->sc, &v, &c->g, c->lb);
      plane_pass(&c->sc, &v, c->lb, &un);
      masked_pass(&c->sc, &v, &c->g, c->lb);
      if (gBoundDecals)
        decal_pass(&c->sc, &v, &c->g, c->lb, &gBoundDecals[(size_t)l * gBoundDecalSlots], gBoundDecalSlots);
    } else {
      for (int i = 0; i < VH * SW; ++i) { c->lb->clip.depth[i] = INFINITY; c->lb->clip.wall[i] = -1; }
    }
    if (unowned) unowned[l] = un;
    if (stages) memcpy(&stages[((size_t)l * 3 + 0) * VH * SW], c->lb->frame, (size_t)VH * SW);
    int nThings = lane[GD_L_THINGS];
    if (nThings > max_things) nThings = max_things;
    if (stage_mask & 2)
      sprite_pass(&c->sc, &v, &c->g, c->lb, &things[(size_t)l * max_things], nThings,
                  depth_override ? &depth_override[(size_t)l * max_things] : NULL);
    if (stages) memcpy(&stages[((size_t)l * 3 + 1) * VH * SW], c->lb->frame, (size_t)VH * SW);
    if (stage_mask & 4) weapon_pass(&c->sc, lane, c->lb->frame);
    if (stages) memcpy(&stages[((size_t)l * 3 + 2) * VH * SW], c->lb->frame, (size_t)VH * SW);
    memcpy(full, c->lb->frame, (size_t)VH * SW);
    if (stage_mask & 8) hud_pass(&c->sc, lane, full + (size_t)VH * SW);
    else memset(full + (size_t)VH * SW, 0, (size_t)GD_HUD_H * SW);
    if (indexed) memcpy(&indexed[(size_t)l * GD_SCREEN_H * SW], full, (size_t)GD_SCREEN_H * SW);
    if (obs) {
      uint8_t pal[768];
      lane_palette(&c->sc, lane, pal);
      area_resize(pal, full, mask_hud ? VH : GD_SCREEN_H, &obs[(size_t)l * GD_OBS * GD_OBS]);
    }
  }
  free(full);
  ctx_free(c);
  return 0;
}

/* PLAYPAL expansion of indexed frames (engine.py:15381-15398); `lanes` (n x 32
 * words, may be NULL) supplies the per-lane screen-flash state. */
int gd_oracle_rgb(const uint8_t *blob, const int32_t *lanes, const uint8_t *indexed, int n, int rows, uint8_t *rgb) {
  Scene sc;
  if (scene_open(&sc, blob) != 0) return -1;
  for (int l = 0; l < n; ++l) {
    uint8_t pal[768];
    lane_palette(&sc, lanes ? &lanes[(size_t)l * GD_LANE_WORDS] : NULL, pal);
    size_t count = (size_t)rows * SW, base = (size_t)l * count;
    for (size_t i = 0; i < count; ++i) memcpy(&rgb[(base + i) * 3], &pal[indexed[base + i] * 3], 3);
  }
  return 0;
}

/* The integer area resize alone, on caller-supplied indexed frames. */
int gd_oracle_resize(const uint8_t *blob, const uint8_t *indexed, int n, int rows, uint8_t *obs) {
  Scene sc;
  if (scene_open(&sc, blob) != 0) return -1;
  for (int l = 0; l < n; ++l)
    area_resize(sc.playpal, &indexed[(size_t)l * rows * SW], rows, &obs[(size_t)l * GD_OBS * GD_OBS]);
  return 0;
}

/* Frame stack update: roll by one and append, or fill all slots for reset
 * lanes (engine.py:9545-9548, 2443-2450).  stack: n x 4 x 84 x 84. */
int gd_oracle_stack(uint8_t *stack, const uint8_t *obs, const uint8_t *reset_mask, int n) {
  size_t fs = (size_t)GD_OBS * GD_OBS;
  for (int l = 0; l < n; ++l) {
    uint8_t *s = &stack[(size_t)l * GD_STACK * fs];
    const uint8_t *o = &obs[(size_t)l * fs];
    if (reset_mask) {
      if (reset_mask[l]) for (int k = 0; k < GD_STACK; ++k) memcpy(s + k * fs, o, fs);
    } else {
      memmove(s, s + fs, (GD_STACK - 1) * fs);
      memcpy(s + (GD_STACK - 1) * fs, o, fs);
    }
  }
  return 0;
}

/* Debug / validation: the complete fallback flat layer of every lane
 * (what engine.py:10956-11171 returns as its frame). out: n x 208 x 320. */
int gd_oracle_flats(const uint8_t *blob, const int32_t *lanes, int n, uint8_t *out) {
  Scene sc;
  if (scene_open(&sc, blob) != 0) return -1;
  FlatLayer *fl = malloc(sizeof(FlatLayer));
  for (int l = 0; l < n; ++l) {
    View v;
    view_setup(&sc, &lanes[(size_t)l * GD_LANE_WORDS], &v);
    flat_layer(&sc, &v, sector_at(&sc, v.x, v.y), fl);
    for (int y = 0; y < VH; ++y)
      for (int x = 0; x < SW; ++x)
        out[((size_t)l * VH + y) * SW + x] = plane_pixel(&sc, &v, fl->sector[y * SW + x], fl->resolved[y * SW + x], x, y);
  }
  free(fl);
  return 0;
}
