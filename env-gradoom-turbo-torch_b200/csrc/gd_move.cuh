/* Per-tic player kinematics (gd_player_tics): one warp per lane.  The 32 threads of a warp
 * carry the same player record through the same control flow; only the loops over the map's
 * walls and sectors are split between them (thread t takes walls t, t + 32, ...) and joined
 * with exact warp reductions (any, float min / max, minimum of (fraction, wall index)), so
 * the result is the serial one.
 * Part of gd_render.cu (one translation unit); not meant to be included elsewhere.
 *
 * Restates src/gradoom/engine.py: _move_player (4344-4575), _doom_axis_slide_move
 * (3207-3498) with _axis_slide_contact_fixed (3120-3205), the box / line and opening
 * tests (2555-2711), _player_actor_collides (2883-2975), _vertical_player_tick
 * (4577-4671) and _sector_at (9598-9617), in the order of one game tic (9558-9573)
 * as far as the player's pose is concerned.  Integer 16.16 / BAM arithmetic on 64-bit
 * integers, float32 where the reference uses it (the library is compiled without
 * fused multiply-add), float64 for the two contact fractions the reference rounds
 * in double precision.
 */
#ifndef GD_MOVE_CUH
#define GD_MOVE_CUH

#define FU 65536LL
#define RADIUS 16.0f
#define RADIUS_FIXED (16LL * FU)
#define PLAYER_HEIGHT 56.0f
#define VIEW_HEIGHT 41.0f
#define U32MASK 0xFFFFFFFFLL

struct GdMoveMap {
  int W, S, nStarts;
  const float *walls;
  const int32_t *wsec, *edgeOff, *edgeWalls, *fineSine;
  const float *secF, *starts;
};

__device__ static i64 gdm_floordiv(i64 a, i64 b) { i64 q = a / b; return ((a % b != 0) && ((a < 0) != (b < 0))) ? q - 1 : q; }
__device__ static i64 gdm_imin(i64 a, i64 b) { return a < b ? a : b; }
__device__ static i64 gdm_imax(i64 a, i64 b) { return a > b ? a : b; }
__device__ static i64 gdm_iclamp(i64 v, i64 lo, i64 hi) { return v < lo ? lo : (v > hi ? hi : v); }
__device__ static i64 gdm_isign(i64 v) { return (v > 0) - (v < 0); }
__device__ static float gdm_fixed_to_float(i64 v) { return (float)v / 65536.0f; }
/* torch.round of a float64: half to even */
__device__ static i64 gdm_round_ratio(i64 numerator, i64 denominator) { return (i64)rint(__ddiv_rn(__dmul_rn((double)numerator, 65536.0), (double)denominator)); }

#define GDM_ALL 0xffffffffu
#define GDM_T ((int)(threadIdx.x & 31))

/* engine.py:9598-9617: the first sector with an odd crossing count; 32 sectors per round */
__device__ static int gdm_sector_at(const GdMoveMap *m, float px, float py) {
  for (int base = 0; base < m->S; base += 32) {
    const int s = base + GDM_T;
    int crossings = 0;
    if (s < m->S)
      for (int k = m->edgeOff[s]; k < m->edgeOff[s + 1]; ++k) {
        const float *e = &m->walls[m->edgeWalls[k] * 4];
        float x1 = e[0], y1 = e[1], x2 = e[2], y2 = e[3];
        int crosses = (y1 > py) != (y2 > py);
        float dy = y2 - y1;
        float safe = fabsf(dy) < 1e-6f ? 1.0f : dy;
        float cx = x1 + (py - y1) * (x2 - x1) / safe;
        crossings += crosses && (px < cx);
      }
    const unsigned odd = __ballot_sync(GDM_ALL, crossings & 1);
    if (odd) return base + __ffs(odd) - 1;
  }
  return 0;
}

/* the actor's box touches the line (engine.py:2568-2598, 2625-2650) */
__device__ static int gdm_box_touches(const float *w, float x, float y, float radius) {
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
__device__ static int gdm_points_collide(const GdMoveMap *m, float x, float y) {
  int hit = 0;
  for (int w = GDM_T; w < m->W; w += 32)
    hit |= m->wsec[w * 2 + 1] < 0 && gdm_box_touches(&m->walls[w * 4], x, y, RADIUS);
  return __any_sync(GDM_ALL, hit);
}

/* engine.py:2600-2711: floor and ceiling under the player's box */
__device__ static void gdm_opening_at(const GdMoveMap *m, float x, float y, float *floorOut, float *ceilOut) {
  int c = gdm_sector_at(m, x, y);
  float floor = m->secF[c * 2], ceiling = m->secF[c * 2 + 1];
  for (int w = GDM_T; w < m->W; w += 32) {
    if (!gdm_box_touches(&m->walls[w * 4], x, y, RADIUS)) continue;
    for (int side = 0; side < 2; ++side) {
      int s = m->wsec[w * 2 + side];
      if (s < 0) continue;
      floor = fmaxf(floor, m->secF[s * 2]);
      ceiling = fminf(ceiling, m->secF[s * 2 + 1]);
    }
  }
  for (int d = 16; d; d >>= 1) {
    floor = fmaxf(floor, __shfl_xor_sync(GDM_ALL, floor, d));
    ceiling = fminf(ceiling, __shfl_xor_sync(GDM_ALL, ceiling, d));
  }
  *floorOut = floor; *ceilOut = ceiling;
}

typedef struct {
  const gd_solid_actors *actors;   /* may be NULL */
  int lane;
} GdmSolids;

__device__ static int gdm_vertical_overlap(float az, float ah, float bz, float bh) { return (az < bz + bh) && (bz < az + ah); }

/* engine.py:2891-2975 */
__device__ static int gdm_actor_collides(const GdMoveMap *m, const GdmSolids *so, float z, float x, float y) {
  const float radius[6] = {20.0f, 20.0f, 16.0f, 20.0f, 30.0f, 24.0f};
  const float height[6] = {56.0f, 56.0f, 56.0f, 56.0f, 56.0f, 64.0f};
  const int noBlock[6] = {10, 10, 20, 10, 20, 24}, xNoBlock[6] = {10, 10, 10, 10, 20, 24};
  const gd_solid_actors *a = so->actors;
  if (a && a->enemy_slots > 0) {
    for (int s = 0; s < a->enemy_slots; ++s) {
      size_t i = (size_t)so->lane * a->enemy_slots + s;
      i64 dt = gdm_iclamp(a->enemy_death_type[i], 0, 5);
      int delay = a->enemy_death_extreme[i] ? xNoBlock[dt] : noBlock[dt];
      int solid = a->enemy_alive[i] ||
                  (a->enemy_death_type[i] >= 0 && a->enemy_death_tics[i] > 0 && a->enemy_death_elapsed[i] < delay);
      if (!solid) continue;
      i64 type = a->enemy_type[i] >= 0 ? a->enemy_type[i] : a->enemy_death_type[i];
      if (type < 0) type = 0;
      if (type > 5) type = 5;
      float h = a->enemy_alive[i] ? height[type] : height[type] * 0.25f;
      if (!gdm_vertical_overlap(z, PLAYER_HEIGHT, a->enemy_z[i], h)) continue;
      if (fabsf(x - a->enemy_x[i]) < RADIUS + radius[type] && fabsf(y - a->enemy_y[i]) < RADIUS + radius[type]) return 1;
    }
  }
  for (int d = 0; d + 1 < m->nStarts; ++d) {      /* voodoo dolls at the unused player starts */
    const float *sp = &m->starts[d * 4];
    if (!gdm_vertical_overlap(z, PLAYER_HEIGHT, sp[3], PLAYER_HEIGHT)) continue;
    if (fabsf(x - sp[0]) < 2 * RADIUS && fabsf(y - sp[1]) < 2 * RADIUS) return 1;
  }
  return 0;
}

/* engine.py:2918-2931 */
__device__ static int gdm_player_collides(const GdMoveMap *m, const GdmSolids *so, float z, float x, float y, float floor, float ceiling) {
  int c = gdm_points_collide(m, x, y);
  c |= floor > z + 24.0f;
  c |= ceiling - fmaxf(z, floor) < 56.0f;
  c |= gdm_actor_collides(m, so, z, x, y);
  return c;
}

typedef struct { i64 fraction; int hitHorizontal, contact; i64 axis; } GdmContact;

/* The serial rule keeps the first blocking wall that reaches the smallest fraction (and the first
 * blocking wall of all when none is valid): the minimum of (fraction, wall index) over the warp. */
__device__ static void gdm_first_smallest(i64 &best, i64 &axis, int &wall) {
  unsigned long long key = ((unsigned long long)best << 32) | (unsigned)wall;
  for (int d = 16; d; d >>= 1) {
    const unsigned long long other = __shfl_xor_sync(GDM_ALL, key, d);
    key = other < key ? other : key;
  }
  wall = (int)(unsigned)key;
  best = (i64)(key >> 32);
  axis = __shfl_sync(GDM_ALL, axis, wall & 31);
  if (wall == 0x7fffffff) { best = FU + 1; axis = 0; }      /* no blocking wall at all */
}

/* engine.py:3120-3205 */
__device__ static GdmContact gdm_axis_contact(const GdMoveMap *m, i64 px, i64 py, i64 mx, i64 my) {
  i64 hBest = FU + 2, vBest = FU + 2, hAxis = 0, vAxis = 0;
  int hWall = 0x7fffffff, vWall = 0x7fffffff;
  i64 safeY = my == 0 ? 1 : my, safeX = mx == 0 ? 1 : mx;
  for (int w = GDM_T; w < m->W; w += 32) {
    if (m->wsec[w * 2 + 1] >= 0) continue;                    /* blocking (one-sided) walls only */
    const float *f = &m->walls[w * 4];
    i64 x1 = (i64)rintf(f[0] * 65536.0f), y1 = (i64)rintf(f[1] * 65536.0f);
    i64 x2 = (i64)rintf(f[2] * 65536.0f), y2 = (i64)rintf(f[3] * 65536.0f);
    {
      i64 target = y1 - gdm_isign(my) * RADIUS_FIXED;
      i64 fraction = gdm_round_ratio(target - py, safeY);
      i64 hx = px + ((mx * fraction) >> 16);
      int valid = (y1 == y2) && my != 0 && fraction >= 0 && fraction <= FU && hx >= gdm_imin(x1, x2) - RADIUS_FIXED &&
                  hx <= gdm_imax(x1, x2) + RADIUS_FIXED;
      i64 cand = valid ? fraction : FU + 1;
      if (cand < hBest) { hBest = cand; hAxis = target; hWall = w; }
    }
    {
      i64 target = x1 - gdm_isign(mx) * RADIUS_FIXED;
      i64 fraction = gdm_round_ratio(target - px, safeX);
      i64 vy = py + ((my * fraction) >> 16);
      int valid = (x1 == x2) && mx != 0 && fraction >= 0 && fraction <= FU && vy >= gdm_imin(y1, y2) - RADIUS_FIXED &&
                  vy <= gdm_imax(y1, y2) + RADIUS_FIXED;
      i64 cand = valid ? fraction : FU + 1;
      if (cand < vBest) { vBest = cand; vAxis = target; vWall = w; }
    }
  }
  gdm_first_smallest(hBest, hAxis, hWall);
  gdm_first_smallest(vBest, vAxis, vWall);
  GdmContact c;
  c.fraction = gdm_imin(hBest, vBest);
  c.hitHorizontal = hBest <= vBest;
  c.contact = c.fraction <= FU;
  c.axis = c.hitHorizontal ? hAxis : vAxis;
  return c;
}

__device__ static i64 gdm_tdiv(i64 a, i64 b) { return a / b; }

/* One game tic of one lane.  `p` is the 32-word player record (enum gd_player_word),
 * `buttons` the tic's button bits (bit i = button i of the reference's button list). */
__device__ static void gdm_player_tic(const GdMoveMap *m, const GdmSolids *so, int32_t *p, uint32_t buttons, int episodeTimeout) {
#define F(word) (*(float *)&p[word])
#define B(i) ((i64)((buttons >> (i)) & 1u))
  const int dead = p[GD_P_FLAGS] & GD_PLAYER_DEAD;
  const int playing = !dead && p[GD_P_EPISODE_TIME] < episodeTimeout;
  if (!playing) buttons = 0;                                   /* active_buttons = buttons & active (9495) */
  /* ---- _move_player (4402-4575) ---- */
  i64 pitch = p[GD_P_PITCH_BAM];
  pitch = gdm_iclamp(pitch - B(17) * (182LL << 16) * playing, -32LL * ((1LL << 29) / 45), 56LL * ((1LL << 29) / 45));
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
  sideMove = gdm_iclamp(sideMove, -(50LL << 11), 50LL << 11);
  if (!onGround) sideMove = (sideMove * 0x0100) >> 16;
  const i64 fine = bam >> 19;
  const i64 sine = m->fineSine[fine], cosine = m->fineSine[(fine + 2048) & 8191];
  const i64 forwardMove = forward * forwardAcc;
  i64 momX = p[GD_P_MOMENTUM_X], momY = p[GD_P_MOMENTUM_Y];
  momX += ((forwardMove * cosine) >> 16) + ((sideMove * sine) >> 16);
  momY += ((forwardMove * sine) >> 16) + ((sideMove * -cosine) >> 16);
  const i64 motionSquared = (momX * momX + momY * momY) >> 16;
  p[GD_P_BOB] = (int32_t)gdm_iclamp((motionSquared * (FU / 4)) >> 16, 0, 16 * FU);

  /* ---- _doom_axis_slide_move (3207-3498) ---- */
  const float z = F(GD_P_Z);
  const i64 startX = p[GD_P_X_FIXED], startY = p[GD_P_Y_FIXED], moveX = momX, moveY = momY;
  const int moved = playing && (moveX != 0 || moveY != 0);
  const i64 dominant = gdm_imax(moveX < 0 ? -moveX : moveX, moveY < 0 ? -moveY : moveY);
  const i64 maxStep = 15 * FU;
  i64 steps = dominant > maxStep ? 1 + gdm_floordiv(dominant, maxStep) : 1;
  if (steps > 3) steps = 3;
  int actorBlocked = 0;
  i64 firstActorStep = 1;
  for (i64 s = 1; s <= 3; ++s) {
    if (s > steps) break;
    i64 sx = startX + gdm_tdiv(moveX * s, steps), sy = startY + gdm_tdiv(moveY * s, steps);
    if (gdm_actor_collides(m, so, z, gdm_fixed_to_float(sx), gdm_fixed_to_float(sy))) { actorBlocked = 1; firstActorStep = s; break; }
  }
  const i64 proposedX = startX + moveX, proposedY = startY + moveY;
  const float pxf = gdm_fixed_to_float(proposedX), pyf = gdm_fixed_to_float(proposedY);
  float proposedFloor, proposedCeiling;
  gdm_opening_at(m, pxf, pyf, &proposedFloor, &proposedCeiling);
  const int blocked = playing && gdm_player_collides(m, so, z, pxf, pyf, proposedFloor, proposedCeiling);
  const int wallBlocked = blocked && gdm_points_collide(m, pxf, pyf);
  const GdmContact full = gdm_axis_contact(m, startX, startY, moveX, moveY);
  i64 collisionStep = gdm_imin(gdm_floordiv(full.fraction * steps, FU) + 1, steps);
  const int actorCollision = playing && actorBlocked && (!full.contact || firstActorStep <= collisionStep);
  const i64 actorPriorX = startX + gdm_tdiv(moveX * (firstActorStep - 1), steps);
  const i64 actorPriorY = startY + gdm_tdiv(moveY * (firstActorStep - 1), steps);
  const i64 oneStepX = gdm_tdiv(moveX, steps), oneStepY = gdm_tdiv(moveY, steps);
  i64 actorPosX = actorPriorX, actorPosY = actorPriorY, actorMomX = 0, actorMomY = 0;
  float actorFloor = F(GD_P_FLOOR_Z), actorCeiling = F(GD_P_CEILING_Z);
  if (actorCollision) {                 /* only then do the actor results reach the output */
    float fy, cy, fx, cx;
    const i64 yx = actorPriorX, yy = actorPriorY + oneStepY, xx = actorPriorX + oneStepX, xy = actorPriorY;
    gdm_opening_at(m, gdm_fixed_to_float(yx), gdm_fixed_to_float(yy), &fy, &cy);
    const int ySucceeds = !gdm_player_collides(m, so, z, gdm_fixed_to_float(yx), gdm_fixed_to_float(yy), fy, cy);
    gdm_opening_at(m, gdm_fixed_to_float(xx), gdm_fixed_to_float(xy), &fx, &cx);
    const int xSucceeds = !ySucceeds && !gdm_player_collides(m, so, z, gdm_fixed_to_float(xx), gdm_fixed_to_float(xy), fx, cx);
    if (ySucceeds) { actorPosX = yx; actorPosY = yy; actorMomX = 0; actorMomY = moveY; actorFloor = fy; actorCeiling = cy; }
    else if (xSucceeds) { actorPosX = xx; actorPosY = xy; actorMomX = moveX; actorMomY = 0; actorFloor = fx; actorCeiling = cx; }
  }
  const i64 priorX = startX + gdm_tdiv(moveX * (collisionStep - 1), steps);
  const i64 priorY = startY + gdm_tdiv(moveY * (collisionStep - 1), steps);
  const GdmContact st = gdm_axis_contact(m, priorX, priorY, oneStepX, oneStepY);
  const int slide = wallBlocked && full.contact && st.contact;
  const i64 approachFraction = gdm_imax(st.fraction - FU / 32, 0);
  const i64 approachX = (oneStepX * approachFraction) >> 16, approachY = (oneStepY * approachFraction) >> 16;
  const i64 remainder = gdm_iclamp(FU - st.fraction, 0, FU);
  const i64 remainingTryX = (oneStepX * remainder) >> 16, remainingTryY = (oneStepY * remainder) >> 16;
  const i64 slideX = st.hitHorizontal ? remainingTryX : 0, slideY = st.hitHorizontal ? 0 : remainingTryY;
  const i64 remainingMoves = 1 + steps - collisionStep;
  const i64 slideTargetX = priorX + approachX + slideX * remainingMoves;
  const i64 slideTargetY = priorY + approachY + slideY * remainingMoves;
  const i64 retryStartX = priorX + approachX, retryStartY = priorY + approachY;
  const i64 retryAxisPosition = st.hitHorizontal ? retryStartY : retryStartX;
  const i64 retryAxisMove = st.hitHorizontal ? remainingTryY : remainingTryX;
  const i64 retryFraction = gdm_round_ratio(st.axis - retryAxisPosition, retryAxisMove == 0 ? 1 : retryAxisMove);
  const int retryGdmContact = retryAxisMove != 0 && retryFraction >= 0 && retryFraction <= FU;
  const i64 retryApproachFraction = gdm_imax(retryFraction - FU / 32, 0);
  const i64 retryApproachX = (remainingTryX * retryApproachFraction) >> 16;
  const i64 retryApproachY = (remainingTryY * retryApproachFraction) >> 16;
  const i64 retryRemainder = gdm_iclamp(FU - retryFraction, 0, FU);
  const i64 retryRemainingX = (remainingTryX * retryRemainder) >> 16, retryRemainingY = (remainingTryY * retryRemainder) >> 16;
  const i64 retrySlideX = st.hitHorizontal ? retryRemainingX : 0, retrySlideY = st.hitHorizontal ? 0 : retryRemainingY;
  const i64 retryTargetX = retryStartX + retryApproachX + retrySlideX * remainingMoves;
  const i64 retryTargetY = retryStartY + retryApproachY + retrySlideY * remainingMoves;
  const int cornerBlocked = slide && gdm_points_collide(m, gdm_fixed_to_float(slideTargetX), gdm_fixed_to_float(slideTargetY));
  const int acceptedSlide = slide && !cornerBlocked;
  const int retrySlide = cornerBlocked && retryGdmContact;
  const int retryBlocked = retrySlide && gdm_points_collide(m, gdm_fixed_to_float(retryTargetX), gdm_fixed_to_float(retryTargetY));
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


struct GdMoveParams {
  GdMoveMap map;
  gd_solid_actors actors;
  int hasActors;
  int32_t *players;
  const uint32_t *buttons;
  int n, tics, episodeTimeout;
  int32_t *lanes;
};

#define GDM_BLOCK 128      /* four lanes per block */

__global__ void __launch_bounds__(GDM_BLOCK) gd_player_tics_kernel(const GdMoveParams q) {
  const int l = (int)(((size_t)blockIdx.x * GDM_BLOCK + threadIdx.x) >> 5);
  if (l >= q.n) return;                                        /* whole warps leave */
  int32_t p[GD_PLAYER_WORDS];
#pragma unroll
  for (int k = 0; k < GD_PLAYER_WORDS; ++k) p[k] = q.players[(size_t)l * GD_PLAYER_WORDS + k];
  GdmSolids so = {q.hasActors ? &q.actors : nullptr, l};
  const uint32_t buttons = q.buttons[l];
  for (int t = 0; t < q.tics; ++t) gdm_player_tic(&q.map, &so, p, buttons, q.episodeTimeout);
  if (GDM_T != 0) return;                                      /* every thread holds the same record */
#pragma unroll
  for (int k = 0; k < GD_PLAYER_WORDS; ++k) q.players[(size_t)l * GD_PLAYER_WORDS + k] = p[k];
  if (q.lanes) {
    /* the pose the renderer reads (src/gradoom/engine.py:4572-4575, 4448, 4410) */
    int32_t *o = q.lanes + (size_t)l * GD_LANE_WORDS;
    const float bamToRad = (float)(2.0 * 3.14159265358979323846 / 4294967296.0);
    o[GD_L_X] = __float_as_int((float)p[GD_P_X_FIXED] / 65536.0f);
    o[GD_L_Y] = __float_as_int((float)p[GD_P_Y_FIXED] / 65536.0f);
    o[GD_L_ANGLE] = __float_as_int((float)(i64)(uint32_t)p[GD_P_ANGLE_BAM] * bamToRad);
    o[GD_L_VIEW_Z] = p[GD_P_VIEW_Z];
    o[GD_L_X_FIXED] = p[GD_P_X_FIXED];
    o[GD_L_Y_FIXED] = p[GD_P_Y_FIXED];
    o[GD_L_ANGLE_BAM] = p[GD_P_ANGLE_BAM];
    o[GD_L_PITCH_BAM] = p[GD_P_PITCH_BAM];
    o[GD_L_BOB_FIXED] = p[GD_P_BOB];
    o[GD_L_EPISODE_TIME] = p[GD_P_EPISODE_TIME];
    o[GD_L_FLAGS] = (o[GD_L_FLAGS] & ~1) | ((p[GD_P_FLAGS] & GD_PLAYER_DEAD) ? 1 : 0);
  }
}

#undef FU
#undef RADIUS
#undef RADIUS_FIXED
#undef PLAYER_HEIGHT
#undef VIEW_HEIGHT
#undef U32MASK
#undef GDM_ALL
#undef GDM_T

extern "C" int gd_player_tics(const gd_renderer *r, int32_t *players, const uint32_t *buttons, const gd_solid_actors *actors,
                              int n, int tics, int episode_timeout, int32_t *lanes, int *status, void *stream) {
  if (!r || !players || !buttons || !status) return GD_ERR_NULL;
  if (n < 0 || tics < 0) return GD_ERR_SIZE;
  if (n == 0 || tics == 0) return GD_OK;
  if (((uintptr_t)players | (uintptr_t)buttons | (uintptr_t)lanes) & 15) return GD_ERR_ALIGN;
  if (actors && actors->enemy_slots > 0) {
    const void *need[] = {actors->enemy_x, actors->enemy_y, actors->enemy_z, actors->enemy_type, actors->enemy_death_type,
                          actors->enemy_death_tics, actors->enemy_death_elapsed, actors->enemy_alive,
                          actors->enemy_death_extreme};
    for (const void *ptr : need) if (!ptr) return GD_ERR_NULL;
  }
  int current = -1;
  if (cudaGetDevice(&current) != cudaSuccess) return GD_ERR_CUDA;
  if (current != r->device) return GD_ERR_DEVICE;
  GdMoveParams q;
  const GdScene &sc = r->sc;
  q.map.W = sc.W; q.map.S = sc.S; q.map.nStarts = r->header[GD_H_STARTS];
  q.map.walls = sc.walls; q.map.wsec = sc.wsec; q.map.edgeOff = sc.edgeOff; q.map.edgeWalls = sc.edgeWalls;
  q.map.fineSine = sc.fineSine; q.map.secF = sc.secF;
  q.map.starts = (const float *)gd_section((const uint8_t *)r->blobDev, r->header, GD_S_STARTS);
  q.hasActors = actors && actors->enemy_slots > 0;
  if (q.hasActors) q.actors = *actors; else memset(&q.actors, 0, sizeof q.actors);
  q.players = players; q.buttons = buttons; q.n = n; q.tics = tics; q.episodeTimeout = episode_timeout; q.lanes = lanes;
  const int lanesPerBlock = GDM_BLOCK / 32;
  gd_player_tics_kernel<<<(n + lanesPerBlock - 1) / lanesPerBlock, GDM_BLOCK, 0, (cudaStream_t)stream>>>(q);
  return cudaGetLastError() == cudaSuccess ? GD_OK : GD_ERR_CUDA;
}

#endif
