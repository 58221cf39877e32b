/* Sprites, the weapon overlay and the status bar.
 * Part of gd_render.cu (one translation unit); not meant to be included elsewhere. */
#ifndef GD_SPRITES_CUH
#define GD_SPRITES_CUH

/* ---- phase: sprites (engine.py:14138-14228, 14684-14947) ----------------- */
__device__ __noinline__ void gd_actor_setup(const GdScene &sc_, const GdView &v_, const gd_thing &t, int sector,
                                            GdActor &ac) {
  const GdScene &sc = *gd_as_shared(&sc_);
  const GdView &v = *gd_as_shared(&v_);
  ac.alive = (t.flags & GD_THING_ALIVE) != 0;
  ac.style = t.style;
  ac.x = t.x; ac.y = t.y;
  int sprite = t.sprite < sc.P ? t.sprite : 0;
  ac.sprite = sprite;
  const int4 si = *reinterpret_cast<const int4 *>(&sc.sprInfo[sprite * 4]);
  ac.w = si.x; ac.h = si.y;
#ifdef GD_CHECKED
  {
    /* a record that names no patch of the scene, or lies nowhere, is not drawn */
    const bool badIndex = t.sprite >= sc.P || si.x > sc.sprW || si.y > sc.sprH || si.x < 0 || si.y < 0;
    const bool badState = !isfinite(t.x) || !isfinite(t.y) || !isfinite(t.z) || sector < 0 || sector >= sc.S;
    if (badIndex) atomicOr(gdCheckedStatus, GD_STATUS_BAD_INDEX);
    if (badState) atomicOr(gdCheckedStatus, GD_STATUS_BAD_STATE);
    if (badIndex || badState) { ac.alive = 0; ac.w = ac.h = 0; if (badState) sector = 0; }
  }
#endif
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
__device__ void gd_sprites(const GdScene &sc_, const GdView &v_, const GdShared &sh_, const GdEvent *events,
                           const int *eventCount, int nThings) {
  const GdScene &sc = *gd_as_shared(&sc_);
  const GdView &v = *gd_as_shared(&v_);
  const GdShared &sh = *gd_as_shared(&sh_);
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
__device__ __noinline__ void gd_weapon_patch(const GdScene &sc_, uint8_t *frame, int id, i64 hoff, i64 voff) {
  frame = gd_as_shared(frame);
  const GdScene &sc = *gd_as_shared(&sc_);
#ifdef GD_CHECKED
  if (id >= sc.Q || id < -1) { if (threadIdx.x == 0) atomicOr(gdCheckedStatus, GD_STATUS_BAD_INDEX); }
#endif
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

__device__ void gd_weapon(const GdScene &sc_, const int32_t *lane, uint8_t *frame) {
  const GdScene &sc = *gd_as_shared(&sc_);
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

struct GdHudList { int4 *entries; int *count; int patches; };

__device__ __forceinline__ void gd_hud_push(const GdHudList &hl, int patch, int x, int y) {
  int n = *hl.count;
#ifdef GD_CHECKED
  if (patch < 0 || patch >= hl.patches) { atomicOr(gdCheckedStatus, GD_STATUS_BAD_INDEX); return; }
#endif
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

__device__ __noinline__ void gd_hud(const GdScene &sc_, const GdShared &sh_, const int32_t *lane, uint8_t *canvas) {
  const GdScene &sc = *gd_as_shared(&sc_);
  const GdShared &sh = *gd_as_shared(&sh_);
  GdHudList hl;
  hl.entries = (int4 *)sh.obs;                       /* free until the resize */
  hl.count = (int *)(sh.obs + GD_HUD_MAX_PATCHES * sizeof(int4));
  hl.patches = sc.hudPatches;
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

#endif
