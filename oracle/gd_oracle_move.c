/*
 * CPU restatement of the reference's per-tic player kinematics: the part of the
 * game dynamics that moves the camera between two renders.
 *
 * TEST INFRASTRUCTURE ONLY (the checker of gd_player_tics in the CUDA library);
 * never called by the product path.
 *
 * Restates, as scalar per-lane C, src/gradoom/engine.py:
 *   turn / thrust / bob                    4344-4575  (_move_player)
 *   wall slide with step-up and openings   3207-3498  (_doom_axis_slide_move)
 *   leading-box contact with axis walls    3120-3205  (_axis_slide_contact_fixed)
 *   box / line tests, openings             2555-2711  (_points_collide, _actor_opening_bounds)
 *   solid actors in the way                2883-2975  (_player_actor_collides and helpers)
 *   view height, gravity, landing          4577-4671  (_vertical_player_tick)
 *   containing sector                      9598-9617  (_sector_at)
 * and the order of one game tic (9558-9573) as far as it concerns the player's pose:
 * weapons, attacks, monsters' thinking and item pickup are not part of it.
 * Pinned on per-tic trajectories recorded from the reference itself
 * (tests/golden/make_golden.py, plan "move").
 * Compile with -ffp-contract=off: every float32 operation is rounded on its own.
 */
#include <math.h>
#include <stdint.h>
#include <string.h>

#include "../include/gradoom_b200.h"

typedef int64_t i64;

#define FU 65536LL
#define RADIUS 16.0f
#define RADIUS_FIXED (16LL * FU)
#define PLAYER_HEIGHT 56.0f
#define VIEW_HEIGHT 41.0f
#define U32MASK 0xFFFFFFFFLL

typedef struct {
  const int32_t *hdr;
  int W, S, nStarts;
  const float *walls;
  const int32_t *wsec, *edgeOff, *edgeWalls, *fineSine;
  const float *secF, *starts;
} Map;

static const void *section(const uint8_t *blob, int s) {
  const int32_t *h = (const int32_t *)blob;
  return blob + h[GD_HDR_SECTION0 + s];
}

static int map_open(Map *m, const uint8_t *blob) {
  const int32_t *h = (const int32_t *)blob;
  if (h[GD_H_MAGIC] != GD_MAGIC || h[GD_H_VERSION] != GD_VERSION) return -1;
  m->hdr = h;
  m->W = h[GD_H_WALLS]; m->S = h[GD_H_SECTORS]; m->nStarts = h[GD_H_STARTS];
  m->walls = section(blob, GD_S_WALLS); m->wsec = section(blob, GD_S_WALL_SECTORS);
  m->edgeOff = section(blob, GD_S_EDGE_OFF); m->edgeWalls = section(blob, GD_S_EDGE_WALLS);
  m->fineSine = section(blob, GD_S_FINESINE); m->secF = section(blob, GD_S_SECTOR_F);
  m->starts = section(blob, GD_S_STARTS);
  return 0;
}

static i64 floordiv(i64 a, i64 b) { i64 q = a / b; return ((a % b != 0) && ((a < 0) != (b < 0))) ? q - 1 : q; }
static i64 imin(i64 a, i64 b) { return a < b ? a : b; }
static i64 imax(i64 a, i64 b) { return a > b ? a : b; }
static i64 iclamp(i64 v, i64 lo, i64 hi) { return v < lo ? lo : (v > hi ? hi : v); }
static i64 isign(i64 v) { return (v > 0) - (v < 0); }
static float fixed_to_float(i64 v) { return (float)v / 65536.0f; }
/* torch.round of a float64: half to even */
static i64 round_ratio(i64 numerator, i64 denominator) { return (i64)rint((double)numerator * 65536.0 / (double)denominator); }

/* engine.py:9598-9617 */
static int sector_at(const Map *m, float px, float py) {
  for (int s = 0; s < m->S; ++s) {
    int crossings = 0;
    for (int k = m->edgeOff[s]; k < m->edgeOff[s + 1]; ++k) {
      const float *e = &m->walls[m->edgeWalls[k] * 4];
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

/* the actor's box touches the line (engine.py:2568-2598, 2625-2650) */
static int box_touches(const float *w, float x, float y, float radius) {
  float left = x - radius, right = x + radius, bottom = y - radius, top = y + radius;
  float x1 = w[0], y1 = w[1], x2 = w[2], y2 = w[3];
  if (!((right > fminf(x1, x2)) && (left < fmaxf(x1, x2)) && (top > fminf(y1, y2)) && (bottom < fmaxf(y1, y2)))) return 0;
  float dx = x2 - x1, dy = y2 - y1;
  float bl = dx * (bottom - y1) - dy * (left - x1);
  float br = dx * (bottom - y1) - dy * (right - x1);
  float tl = dx * (top - y1) - dy * (left - x1);
  float tr = dx * (top - y1) - dy * (right - x1);
  float lo = fminf(fminf(bl, br), fminf(tl, tr)), hi = fmaxf(fmaxf(bl, br), fmaxf(tl, tr));
  return lo <= 0 && hi >= 0;
}

/* engine.py:2555-2598: any one-sided wall crosses the player's box */
static int points_collide(const Map *m, float x, float y) {
  for (int w = 0; w < m->W; ++w)
    if (m->wsec[w * 2 + 1] < 0 && box_touches(&m->walls[w * 4], x, y, RADIUS)) return 1;
  return 0;
}

/* engine.py:2600-2711: floor and ceiling under the player's box */
static void opening_at(const Map *m, float x, float y, float *floorOut, float *ceilOut) {
  int c = sector_at(m, x, y);
  float floor = m->secF[c * 2], ceiling = m->secF[c * 2 + 1];
  for (int w = 0; w < m->W; ++w) {
    if (!box_touches(&m->walls[w * 4], x, y, RADIUS)) continue;
    for (int side = 0; side < 2; ++side) {
      int s = m->wsec[w * 2 + side];
      if (s < 0) continue;
      floor = fmaxf(floor, m->secF[s * 2]);
      ceiling = fminf(ceiling, m->secF[s * 2 + 1]);
    }
  }
  *floorOut = floor; *ceilOut = ceiling;
}

typedef struct {
  const gd_solid_actors *actors;   /* may be NULL */
  int lane;
} Solids;

static int vertical_overlap(float az, float ah, float bz, float bh) { return (az < bz + bh) && (bz < az + ah); }

/* engine.py:2891-2975 */
static int actor_collides(const Map *m, const Solids *so, float z, float x, float y) {
  static const float radius[6] = {20.0f, 20.0f, 16.0f, 20.0f, 30.0f, 24.0f};
  static const float height[6] = {56.0f, 56.0f, 56.0f, 56.0f, 56.0f, 64.0f};
  static const int noBlock[6] = {10, 10, 20, 10, 20, 24}, xNoBlock[6] = {10, 10, 10, 10, 20, 24};
  const gd_solid_actors *a = so->actors;
  if (a && a->enemy_slots > 0) {
    for (int s = 0; s < a->enemy_slots; ++s) {
      size_t i = (size_t)so->lane * a->enemy_slots + s;
      i64 dt = iclamp(a->enemy_death_type[i], 0, 5);
      int delay = a->enemy_death_extreme[i] ? xNoBlock[dt] : noBlock[dt];
      int solid = a->enemy_alive[i] ||
                  (a->enemy_death_type[i] >= 0 && a->enemy_death_tics[i] > 0 && a->enemy_death_elapsed[i] < delay);
      if (!solid) continue;
      i64 type = a->enemy_type[i] >= 0 ? a->enemy_type[i] : a->enemy_death_type[i];
      if (type < 0) type = 0;
      if (type > 5) type = 5;
      float h = a->enemy_alive[i] ? height[type] : height[type] * 0.25f;
      if (!vertical_overlap(z, PLAYER_HEIGHT, a->enemy_z[i], h)) continue;
      if (fabsf(x - a->enemy_x[i]) < RADIUS + radius[type] && fabsf(y - a->enemy_y[i]) < RADIUS + radius[type]) return 1;
    }
  }
  for (int d = 0; d + 1 < m->nStarts; ++d) {      /* voodoo dolls at the unused player starts */
    const float *sp = &m->starts[d * 4];
    if (!vertical_overlap(z, PLAYER_HEIGHT, sp[3], PLAYER_HEIGHT)) continue;
    if (fabsf(x - sp[0]) < 2 * RADIUS && fabsf(y - sp[1]) < 2 * RADIUS) return 1;
  }
  return 0;
}

/* engine.py:2918-2931 */
static int player_collides(const Map *m, const Solids *so, float z, float x, float y, float floor, float ceiling) {
  int c = points_collide(m, x, y);
  c |= floor > z + 24.0f;
  c |= ceiling - fmaxf(z, floor) < 56.0f;
  c |= actor_collides(m, so, z, x, y);
  return c;
}

typedef struct { i64 fraction; int hitHorizontal, contact; i64 axis; } Contact;

/* engine.py:3120-3205 */
static Contact axis_contact(const Map *m, i64 px, i64 py, i64 mx, i64 my) {
  i64 hBest = FU + 1, vBest = FU + 1, hAxis = 0, vAxis = 0;
  int hFirst = 1, vFirst = 1;
  i64 safeY = my == 0 ? 1 : my, safeX = mx == 0 ? 1 : mx;
  for (int w = 0; w < m->W; ++w) {
    if (m->wsec[w * 2 + 1] >= 0) continue;                    /* blocking (one-sided) walls only */
    const float *f = &m->walls[w * 4];
    i64 x1 = (i64)rintf(f[0] * 65536.0f), y1 = (i64)rintf(f[1] * 65536.0f);
    i64 x2 = (i64)rintf(f[2] * 65536.0f), y2 = (i64)rintf(f[3] * 65536.0f);
    {
      i64 target = y1 - isign(my) * RADIUS_FIXED;
      i64 fraction = round_ratio(target - py, safeY);
      i64 hx = px + ((mx * fraction) >> 16);
      int valid = (y1 == y2) && my != 0 && fraction >= 0 && fraction <= FU && hx >= imin(x1, x2) - RADIUS_FIXED &&
                  hx <= imax(x1, x2) + RADIUS_FIXED;
      i64 cand = valid ? fraction : FU + 1;
      if (hFirst || cand < hBest) { hBest = cand; hAxis = target; hFirst = 0; }
    }
    {
      i64 target = x1 - isign(mx) * RADIUS_FIXED;
      i64 fraction = round_ratio(target - px, safeX);
      i64 vy = py + ((my * fraction) >> 16);
      int valid = (x1 == x2) && mx != 0 && fraction >= 0 && fraction <= FU && vy >= imin(y1, y2) - RADIUS_FIXED &&
                  vy <= imax(y1, y2) + RADIUS_FIXED;
      i64 cand = valid ? fraction : FU + 1;
      if (vFirst || cand < vBest) { vBest = cand; vAxis = target; vFirst = 0; }
    }
  }
  Contact c;
  c.fraction = imin(hBest, vBest);
  c.hitHorizontal = hBest <= vBest;
  c.contact = c.fraction <= FU;
  c.axis = c.hitHorizontal ? hAxis : vAxis;
  return c;
}

static i64 tdiv(i64 a, i64 b) { return a / b; }

/* One game tic of one lane.  `p` is the 32-word player record (enum gd_player_word),
 * `buttons` the tic's button bits (bit i = button i of the reference's button list). */
static void player_tic(const Map *m, const Solids *so, int32_t *p, uint32_t buttons, int episodeTimeout) {
#define F(word) (*(float *)&p[word])
#define B(i) ((i64)((buttons >> (i)) & 1u))
  const int dead = p[GD_P_FLAGS] & GD_PLAYER_DEAD;
  const int playing = !dead && p[GD_P_EPISODE_TIME] < episodeTimeout;
  if (!playing) buttons = 0;                                   /* active_buttons = buttons & active (9495) */
  /* ---- _move_player (4402-4575) ---- */
  i64 pitch = p[GD_P_PITCH_BAM];
  pitch = iclamp(pitch - B(17) * (182LL << 16) * playing, -32LL * ((1LL << 29) / 45), 56LL * ((1LL << 29) / 45));
  p[GD_P_PITCH_BAM] = (int32_t)pitch;
  const int active = p[GD_P_REACTION_TIME] <= 0 && playing;
  const int pullRequested = ((p[GD_P_FLAGS] & GD_PLAYER_CHAINSAW_PULL) != 0) && playing;
  const int pullActive = pullRequested && active;
  if (pullRequested) p[GD_P_FLAGS] &= ~GD_PLAYER_CHAINSAW_PULL;
  p[GD_P_REACTION_TIME] = p[GD_P_REACTION_TIME] - 1 < 0 ? 0 : p[GD_P_REACTION_TIME] - 1;
  const float currentFloor = F(GD_P_FLOOR_Z);
  F(GD_P_PREV_FLOOR_Z) = currentFloor;
  const int onGround = F(GD_P_Z) <= currentFloor;
  const int turning = B(7) | B(8);
  p[GD_P_TURN_HELD] = turning ? p[GD_P_TURN_HELD] + 1 : 0;
  const i64 yaw = p[GD_P_TURN_HELD] < 6 ? 320 : (B(1) ? 1280 : 640);
  const i64 turnDirection = B(8) - B(7);
  const i64 keyboardTurn = active && !pullRequested && !B(2), deltaTurn = active && !pullRequested;
  i64 turnDelta = ((turnDirection * yaw) << 16) * keyboardTurn;
  turnDelta -= ((B(18) * 182) << 16) * deltaTurn;
  const i64 bam = ((i64)(uint32_t)p[GD_P_ANGLE_BAM] + turnDelta) & U32MASK;
  p[GD_P_ANGLE_BAM] = (int32_t)(uint32_t)bam;
  i64 forward = (B(6) - B(5)) * active;
  i64 side = (B(3) - B(4)) + B(2) * (B(7) - B(8));
  side *= active;
  if (pullActive) forward = 1;
  if (pullRequested) side = 0;
  i64 forwardAcc = B(1) ? (50LL << 11) : (25LL << 11);
  if (pullActive) forwardAcc = 100LL << 11;
  const i64 sideAcc = B(1) ? (40LL << 11) : (24LL << 11);
  if (!onGround) forwardAcc = (forwardAcc * 0x0100) >> 16;
  i64 sideMove = side * sideAcc + B(19) * (1LL << 11) * active;
  if (pullRequested) sideMove = 0;
  sideMove = iclamp(sideMove, -(50LL << 11), 50LL << 11);
  if (!onGround) sideMove = (sideMove * 0x0100) >> 16;
  const i64 fine = bam >> 19;
  const i64 sine = m->fineSine[fine], cosine = m->fineSine[(fine + 2048) & 8191];
  const i64 forwardMove = forward * forwardAcc;
  i64 momX = p[GD_P_MOMENTUM_X], momY = p[GD_P_MOMENTUM_Y];
  momX += ((forwardMove * cosine) >> 16) + ((sideMove * sine) >> 16);
  momY += ((forwardMove * sine) >> 16) + ((sideMove * -cosine) >> 16);
  const i64 motionSquared = (momX * momX + momY * momY) >> 16;
  p[GD_P_BOB] = (int32_t)iclamp((motionSquared * (FU / 4)) >> 16, 0, 16 * FU);

  /* ---- _doom_axis_slide_move (3207-3498) ---- */
  const float z = F(GD_P_Z);
  const i64 startX = p[GD_P_X_FIXED], startY = p[GD_P_Y_FIXED], moveX = momX, moveY = momY;
  const int moved = playing && (moveX != 0 || moveY != 0);
  const i64 dominant = imax(moveX < 0 ? -moveX : moveX, moveY < 0 ? -moveY : moveY);
  const i64 maxStep = 15 * FU;
  i64 steps = dominant > maxStep ? 1 + floordiv(dominant, maxStep) : 1;
  if (steps > 3) steps = 3;
  int actorBlocked = 0;
  i64 firstActorStep = 1;
  for (i64 s = 1; s <= 3; ++s) {
    if (s > steps) break;
    i64 sx = startX + tdiv(moveX * s, steps), sy = startY + tdiv(moveY * s, steps);
    if (actor_collides(m, so, z, fixed_to_float(sx), fixed_to_float(sy))) { actorBlocked = 1; firstActorStep = s; break; }
  }
  const i64 proposedX = startX + moveX, proposedY = startY + moveY;
  const float pxf = fixed_to_float(proposedX), pyf = fixed_to_float(proposedY);
  float proposedFloor, proposedCeiling;
  opening_at(m, pxf, pyf, &proposedFloor, &proposedCeiling);
  const int blocked = playing && player_collides(m, so, z, pxf, pyf, proposedFloor, proposedCeiling);
  const int wallBlocked = blocked && points_collide(m, pxf, pyf);
  const Contact full = axis_contact(m, startX, startY, moveX, moveY);
  i64 collisionStep = imin(floordiv(full.fraction * steps, FU) + 1, steps);
  const int actorCollision = playing && actorBlocked && (!full.contact || firstActorStep <= collisionStep);
  const i64 actorPriorX = startX + tdiv(moveX * (firstActorStep - 1), steps);
  const i64 actorPriorY = startY + tdiv(moveY * (firstActorStep - 1), steps);
  const i64 oneStepX = tdiv(moveX, steps), oneStepY = tdiv(moveY, steps);
  i64 actorPosX = actorPriorX, actorPosY = actorPriorY, actorMomX = 0, actorMomY = 0;
  float actorFloor = F(GD_P_FLOOR_Z), actorCeiling = F(GD_P_CEILING_Z);
  if (actorCollision) {                 /* only then do the actor results reach the output */
    float fy, cy, fx, cx;
    const i64 yx = actorPriorX, yy = actorPriorY + oneStepY, xx = actorPriorX + oneStepX, xy = actorPriorY;
    opening_at(m, fixed_to_float(yx), fixed_to_float(yy), &fy, &cy);
    const int ySucceeds = !player_collides(m, so, z, fixed_to_float(yx), fixed_to_float(yy), fy, cy);
    opening_at(m, fixed_to_float(xx), fixed_to_float(xy), &fx, &cx);
    const int xSucceeds = !ySucceeds && !player_collides(m, so, z, fixed_to_float(xx), fixed_to_float(xy), fx, cx);
    if (ySucceeds) { actorPosX = yx; actorPosY = yy; actorMomX = 0; actorMomY = moveY; actorFloor = fy; actorCeiling = cy; }
    else if (xSucceeds) { actorPosX = xx; actorPosY = xy; actorMomX = moveX; actorMomY = 0; actorFloor = fx; actorCeiling = cx; }
  }
  const i64 priorX = startX + tdiv(moveX * (collisionStep - 1), steps);
  const i64 priorY = startY + tdiv(moveY * (collisionStep - 1), steps);
  const Contact st = axis_contact(m, priorX, priorY, oneStepX, oneStepY);
  const int slide = wallBlocked && full.contact && st.contact;
  const i64 approachFraction = imax(st.fraction - FU / 32, 0);
  const i64 approachX = (oneStepX * approachFraction) >> 16, approachY = (oneStepY * approachFraction) >> 16;
  const i64 remainder = iclamp(FU - st.fraction, 0, FU);
  const i64 remainingTryX = (oneStepX * remainder) >> 16, remainingTryY = (oneStepY * remainder) >> 16;
  const i64 slideX = st.hitHorizontal ? remainingTryX : 0, slideY = st.hitHorizontal ? 0 : remainingTryY;
  const i64 remainingMoves = 1 + steps - collisionStep;
  const i64 slideTargetX = priorX + approachX + slideX * remainingMoves;
  const i64 slideTargetY = priorY + approachY + slideY * remainingMoves;
  const i64 retryStartX = priorX + approachX, retryStartY = priorY + approachY;
  const i64 retryAxisPosition = st.hitHorizontal ? retryStartY : retryStartX;
  const i64 retryAxisMove = st.hitHorizontal ? remainingTryY : remainingTryX;
  const i64 retryFraction = round_ratio(st.axis - retryAxisPosition, retryAxisMove == 0 ? 1 : retryAxisMove);
  const int retryContact = retryAxisMove != 0 && retryFraction >= 0 && retryFraction <= FU;
  const i64 retryApproachFraction = imax(retryFraction - FU / 32, 0);
  const i64 retryApproachX = (remainingTryX * retryApproachFraction) >> 16;
  const i64 retryApproachY = (remainingTryY * retryApproachFraction) >> 16;
  const i64 retryRemainder = iclamp(FU - retryFraction, 0, FU);
  const i64 retryRemainingX = (remainingTryX * retryRemainder) >> 16, retryRemainingY = (remainingTryY * retryRemainder) >> 16;
  const i64 retrySlideX = st.hitHorizontal ? retryRemainingX : 0, retrySlideY = st.hitHorizontal ? 0 : retryRemainingY;
  const i64 retryTargetX = retryStartX + retryApproachX + retrySlideX * remainingMoves;
  const i64 retryTargetY = retryStartY + retryApproachY + retrySlideY * remainingMoves;
  const int cornerBlocked = slide && points_collide(m, fixed_to_float(slideTargetX), fixed_to_float(slideTargetY));
  const int acceptedSlide = slide && !cornerBlocked;
  const int retrySlide = cornerBlocked && retryContact;
  const int retryBlocked = retrySlide && points_collide(m, fixed_to_float(retryTargetX), fixed_to_float(retryTargetY));
  const int acceptedRetry = retrySlide && !retryBlocked;
  const int stalledRetry = cornerBlocked && (!retrySlide || retryBlocked);
  i64 posX = acceptedSlide ? slideTargetX : (acceptedRetry ? retryTargetX : (stalledRetry ? retryStartX + retryApproachX : proposedX));
  i64 posY = acceptedSlide ? slideTargetY : (acceptedRetry ? retryTargetY : (stalledRetry ? retryStartY + retryApproachY : proposedY));
  i64 resultMoveX = slide ? (retrySlide ? retrySlideX : slideX) * steps : moveX;
  i64 resultMoveY = slide ? (retrySlide ? retrySlideY : slideY) * steps : moveY;
  if (actorCollision) { posX = actorPosX; posY = actorPosY; resultMoveX = actorMomX; resultMoveY = actorMomY; }
  if (!playing) { posX = startX; posY = startY; }
  const int fallback = blocked && !slide && !actorCollision;
  const int preserveOpening = blocked || !moved;
  float resultFloor = preserveOpening ? F(GD_P_FLOOR_Z) : proposedFloor;
  float resultCeiling = preserveOpening ? F(GD_P_CEILING_Z) : proposedCeiling;
  if (actorCollision) { resultFloor = actorFloor; resultCeiling = actorCeiling; }
  /* back in _move_player (4539-4575) */
  if (!fallback) { p[GD_P_X_FIXED] = (int32_t)posX; p[GD_P_Y_FIXED] = (int32_t)posY; }
  const i64 nextMomX = fallback ? 0 : resultMoveX, nextMomY = fallback ? 0 : resultMoveY;
  F(GD_P_FLOOR_Z) = resultFloor;
  F(GD_P_CEILING_Z) = resultCeiling;
  const i64 friction = z <= resultFloor ? 0xE800 : FU;
  p[GD_P_MOMENTUM_X] = (int32_t)((nextMomX * friction) >> 16);
  p[GD_P_MOMENTUM_Y] = (int32_t)((nextMomY * friction) >> 16);

  /* ---- _vertical_player_tick (4577-4671), active = the tic's `active` (9435) ---- */
  if (playing) {
    float viewHeight = F(GD_P_VIEW_HEIGHT), deltaVH = F(GD_P_DELTA_VIEW_HEIGHT), velocityZ = F(GD_P_VELOCITY_Z);
    float nextVH = viewHeight + deltaVH;
    const int above = nextVH > VIEW_HEIGHT, below = nextVH < VIEW_HEIGHT / 2.0f;
    nextVH = above ? VIEW_HEIGHT : (below ? VIEW_HEIGHT / 2.0f : nextVH);
    float nextDelta = above ? 0.0f : deltaVH;
    if (below && nextDelta <= 0) nextDelta = 1.0f / 65536.0f;
    const int movingView = nextDelta != 0;
    if (movingView) nextDelta = nextDelta + 0.25f;
    if (movingView && nextDelta == 0) nextDelta = 1.0f / 65536.0f;
    const i64 bobAngle = (((i64)p[GD_P_EPISODE_TIME] * 8192) / 20) & 8191;
    const i64 viewBob = (((i64)p[GD_P_BOB] >> 1) * m->fineSine[bobAngle]) >> 16;
    float nextViewZ = z + nextVH + (float)viewBob / 65536.0f;
    nextViewZ = fminf(nextViewZ, resultCeiling - 4.0f);
    nextViewZ = fmaxf(nextViewZ, resultFloor + 4.0f);
    F(GD_P_VIEW_Z) = nextViewZ;
    const float floor = resultFloor;
    const int smoothStepUp = z < floor;
    const float steppedVH = nextVH - (floor - z);
    if (smoothStepUp) { nextVH = steppedVH; nextDelta = (VIEW_HEIGHT - steppedVH) / 8.0f; }
    const float proposedZ = z + velocityZ;
    const int airborne = (z > floor) || (velocityZ < 0);
    const float previousFloor = F(GD_P_PREV_FLOOR_Z);
    const int walkedOffLedge = velocityZ == 0 && previousFloor > floor && proposedZ == previousFloor;
    const float gravity = walkedOffLedge ? 2.0f : 1.0f;
    float nextVelocity = airborne ? velocityZ - gravity : 0.0f;
    const int landed = proposedZ <= floor;
    const float nextZ = landed ? floor : proposedZ;
    if (landed && airborne && velocityZ < -8.0f) nextDelta = velocityZ / 8.0f;
    if (landed) nextVelocity = 0.0f;
    F(GD_P_VIEW_HEIGHT) = nextVH;
    F(GD_P_Z) = nextZ;
    F(GD_P_VELOCITY_Z) = nextVelocity;
    F(GD_P_DELTA_VIEW_HEIGHT) = nextDelta;
    p[GD_P_EPISODE_TIME] += 1;                                 /* episode_time += active (9572) */
  }
#undef F
#undef B
}

/* Advance n lanes by `tics` game tics with the same buttons each (one agent step with
 * frame skip `tics`).  players: n x GD_PLAYER_WORDS; buttons: n button masks. */
int gd_oracle_player_tics(const uint8_t *blob, int32_t *players, const uint32_t *buttons, const gd_solid_actors *actors,
                          int n, int tics, int episode_timeout) {
  Map m;
  if (map_open(&m, blob) != 0) return -1;
  for (int l = 0; l < n; ++l) {
    Solids so = {actors, l};
    for (int t = 0; t < tics; ++t) player_tic(&m, &so, players + (size_t)l * GD_PLAYER_WORDS, buttons[l], episode_timeout);
  }
  return 0;
}
