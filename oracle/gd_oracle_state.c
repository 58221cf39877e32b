/*
 * CPU restatement of the step between the reference engine's lane tensors and
 * the renderer's inputs: the lane records and the thing records.
 *
 * TEST INFRASTRUCTURE ONLY (the checker of gd_pack_state in the CUDA library and
 * the packer the fixture generator uses on a machine without a GPU); never
 * called by the product path.
 *
 * Restates, as scalar loops over lanes and slots, src/gradoom/engine.py:
 *   view pose selection        2122-2133 (_public_or_retained_fixed), 10648-10658
 *   active weapon              4673-4676
 *   sprite rotation            13994-14009
 *   enemy sprite ids           14011-14077
 *   corpse sprite ids          14079-14104
 *   explosion sprite ids       14106-14122
 *   enemy full-bright states   14124-14136
 *   map item sprite ids        14258-14317
 *   actor concatenation order  14328-14682
 * Compile with -ffp-contract=off: every float32 operation is rounded on its own.
 */
#include <math.h>
#include <stdint.h>
#include <string.h>

#include "../include/gradoom_b200.h"

typedef int64_t i64;

static const int kWalkTics[6] = {8, 6, 4, 6, 4, 6};
static const int kIdleTics[6] = {10, 10, 8, 10, 10, 10};
static const int kRecovery[6] = {16, 20, 4, 4, 8, 8};
static const int kSlotBaseWeapon[7] = {0, 0, 2, 3, 5, 6, 7};

static const void *section(const uint8_t *blob, int s) {
  const int32_t *h = (const int32_t *)blob;
  return blob + h[GD_HDR_SECTION0 + s];
}

static int32_t fbits(float f) { int32_t i; memcpy(&i, &f, 4); return i; }
static i64 floordiv(i64 a, i64 b) { i64 q = a / b; return ((a % b != 0) && ((a < 0) != (b < 0))) ? q - 1 : q; }
static i64 pymod(i64 a, i64 m) { i64 r = a % m; return (r != 0 && ((r < 0) != (m < 0))) ? r + m : r; }
static float pyfmodf(float a, float b) { float r = fmodf(a, b); return (r != 0.0f && ((b < 0) != (r < 0))) ? r + b : r; }
static int clampi(i64 v, int lo, int hi) { return v < lo ? lo : (v > hi ? hi : (int)v); }

/* engine.py:13994-14009 */
static int rotation(float viewer, float actor) {
  const float eighth = (float)(M_PI / 8), twoPi = (float)(2 * M_PI), quarter = (float)(M_PI / 4);
  float relative = pyfmodf(viewer - actor + eighth, twoPi);
  return (int)pymod((i64)floorf(relative / quarter), 8);
}

static int frame_from_ends(i64 elapsed, const int32_t *ends, int frames, int count) {
  int f = 0;
  for (int k = 0; k < frames; ++k) f += elapsed >= ends[k];
  f = f < count - 1 ? f : count - 1;
  return (int)pymod(f, frames);    /* an empty animation indexes from the end, as the tensor lookup does */
}

typedef struct { const uint8_t *blob; const gd_engine_state *st; int32_t *things; int maxThings, K, pos; } Emit;

static void put(Emit *e, int lane, float x, float y, float z, int sprite, int alive, int bright, int style) {
  if (e->pos >= e->maxThings) return;
  int32_t *t = e->things + ((size_t)lane * (e->maxThings > 0 ? e->maxThings : 1) + e->pos) * 4;
  t[0] = fbits(x); t[1] = fbits(y); t[2] = fbits(z);
  uint32_t word = ((uint32_t)sprite & 0xFFFFu) | ((uint32_t)((alive ? GD_THING_ALIVE : 0) | (bright ? GD_THING_BRIGHT : 0)) << 16) |
                  (((uint32_t)style & 0xFFu) << 24);
  t[3] = (int32_t)word;
}

/* Returns K, the number of records every lane gets (it may exceed max_things; the
 * records beyond are not written). */
int gd_oracle_pack_state(const uint8_t *blob, const gd_engine_state *st, int max_things, int32_t *lanes, int32_t *things) {
  const int32_t *h = (const int32_t *)blob;
  if (h[GD_H_MAGIC] != GD_MAGIC || h[GD_H_VERSION] != GD_VERSION) return -1;
  const int n = st->n, E = st->enemy_slots, PP = st->projectile_slots, EP = st->enemy_projectile_slots,
            PF = st->puff_slots, I = st->items;
  const int32_t *walk = section(blob, GD_S_ENEMY_WALK), *attack = section(blob, GD_S_ENEMY_ATTACK),
                *pain = section(blob, GD_S_ENEMY_PAIN), *deathIds = section(blob, GD_S_DEATH_IDS),
                *deathCounts = section(blob, GD_S_DEATH_COUNTS), *deathEnds = section(blob, GD_S_DEATH_ENDS),
                *xdeathIds = section(blob, GD_S_XDEATH_IDS), *xdeathCounts = section(blob, GD_S_XDEATH_COUNTS),
                *xdeathEnds = section(blob, GD_S_XDEATH_ENDS), *flight = section(blob, GD_S_PROJ_FLIGHT),
                *explIds = section(blob, GD_S_PROJ_EXPL_IDS), *explCounts = section(blob, GD_S_PROJ_EXPL_COUNTS),
                *explEnds = section(blob, GD_S_PROJ_EXPL_ENDS), *explTotal = section(blob, GD_S_PROJ_EXPL_TOTAL),
                *fogIds = section(blob, GD_S_FOG_IDS), *puffIds = section(blob, GD_S_PUFF_IDS),
                *staticIds = section(blob, GD_S_STATIC_IDS), *itemInfo = section(blob, GD_S_ITEM_INFO),
                *itemAnim = section(blob, GD_S_ITEM_ANIM);
  const float *starts = section(blob, GD_S_STARTS), *itemPos = section(blob, GD_S_ITEM_POS);
  const int dolls = h[GD_H_STARTS] > 0 ? h[GD_H_STARTS] - 1 : 0;
  const int DF = h[GD_H_DEATH_FRAMES], XF = h[GD_H_XDEATH_FRAMES];
  if (I != h[GD_H_ITEMS]) return -2;

  /* slots of each class that some lane of the batch uses */
  enum { ENEMY, CORPSE, PFLIGHT, EFLIGHT, PIMPACT, EIMPACT, FOG, PUFF, ITEM, DROP, CLASSES };
  static uint8_t used[CLASSES][4096];
  memset(used, 0, sizeof used);
  if (E > 4096 || PP > 4096 || EP > 4096 || PF > 4096 || I > 4096) return -3;
  for (int l = 0; l < n; ++l) {
    for (int s = 0; s < E; ++s) {
      size_t i = (size_t)l * E + s;
      used[ENEMY][s] |= st->enemy_alive[i] != 0;
      used[CORPSE][s] |= st->enemy_death_tics[i] > 0;
      used[FOG][s] |= st->teleport_fog_tics[i] > 0;
      used[DROP][s] |= (st->drop_type[i] >= 0) && st->drop_spawned[i];
    }
    for (int s = 0; s < PP; ++s) {
      size_t i = (size_t)l * PP + s;
      used[PFLIGHT][s] |= st->projectile_alive[i] != 0;
      used[PIMPACT][s] |= st->projectile_impact_tics[i] > 0;
    }
    for (int s = 0; s < EP; ++s) {
      size_t i = (size_t)l * EP + s;
      used[EFLIGHT][s] |= st->enemy_projectile_alive[i] != 0;
      used[EIMPACT][s] |= st->enemy_projectile_impact_tics[i] > 0;
    }
    for (int s = 0; s < PF; ++s) used[PUFF][s] |= st->hitscan_puff_tics[(size_t)l * PF + s] > 0;
    for (int s = 0; s < I; ++s) used[ITEM][s] |= st->item_available[(size_t)l * I + s] != 0;
  }

  int K = 0;
  for (int l = 0; l < n; ++l) {
    Emit e = {blob, st, things, max_things, 0, 0};
    const float px = st->x[l], py = st->y[l];
    /* living enemies (engine.py:14330-14343, 14011-14077, 14124-14136) */
    for (int s = 0; s < E; ++s) {
      if (!used[ENEMY][s]) continue;
      size_t i = (size_t)l * E + s;
      int type = clampi(st->enemy_type[i], 0, 5);
      float viewer = atan2f(py - st->enemy_y[i], px - st->enemy_x[i]);
      int rot = rotation(viewer, st->enemy_angle[i]);
      i64 tics = st->enemy_animation_tics[i];
      int walkFrame = (int)pymod(floordiv(tics, kWalkTics[type]), 4);
      int idleFrame = (int)pymod(floordiv(tics, kIdleTics[type]), 2);
      if (type == 2) idleFrame = 0;
      if (st->enemy_target_slot[i] < -1) walkFrame = idleFrame;
      int phase = st->enemy_attack_phase[i], cooldown = st->enemy_cooldown[i];
      int recovering = cooldown > (kRecovery[type] / 2);
      int attackFrame = 0;
      if (type == 0 || type == 1) attackFrame = phase == 2 ? recovering : 0;
      if ((type == 4 || type == 5) && phase == 1) attackFrame = cooldown <= 8;
      if ((type == 4 || type == 5) && phase == 2) attackFrame = 2;
      if (type == 3 && (phase == 4 || phase == 2)) attackFrame = 1;
      if (type == 3 && phase == 3) attackFrame = 2;
      int sprite = phase > 0 ? attack[(type * 4 + attackFrame) * 8 + rot] : walk[(type * 4 + walkFrame) * 8 + rot];
      if (st->enemy_pain_tics[i] > 0) sprite = pain[type * 8 + rot];
      int bright = (type == 1 && phase == 2 && recovering) || (type == 3 && (phase == 2 || phase == 3));
      put(&e, l, st->enemy_x[i], st->enemy_y[i], st->enemy_z[i], sprite, st->enemy_alive[i] != 0, bright, -1);
      e.pos++;
    }
    /* voodoo dolls at the unused player starts (14345-14381) */
    for (int d = 0; d < dolls; ++d) {
      const float *sp = &starts[d * 4];
      float viewer = atan2f(py - sp[1], px - sp[0]);
      int rot = rotation(viewer, sp[2]);
      put(&e, l, sp[0], sp[1], sp[3], walk[(2 * 4 + 0) * 8 + rot], !st->player_dead[l], 0, -1);
      e.pos++;
    }
    /* corpses (14383-14410, 14079-14104) */
    for (int s = 0; s < E; ++s) {
      if (!used[CORPSE][s]) continue;
      size_t i = (size_t)l * E + s;
      int type = clampi(st->enemy_death_type[i], 0, 5);
      i64 elapsed = st->enemy_death_elapsed[i];
      int sprite = st->enemy_death_extreme[i]
                       ? xdeathIds[type * XF + frame_from_ends(elapsed, &xdeathEnds[type * XF], XF, xdeathCounts[type])]
                       : deathIds[type * DF + frame_from_ends(elapsed, &deathEnds[type * DF], DF, deathCounts[type])];
      put(&e, l, st->enemy_x[i], st->enemy_y[i], st->enemy_z[i], sprite, st->enemy_death_tics[i] > 0, 0, -1);
      e.pos++;
    }
    /* player projectiles in flight (14412-14460) */
    for (int s = 0; s < PP; ++s) {
      if (!used[PFLIGHT][s]) continue;
      size_t i = (size_t)l * PP + s;
      int type = clampi(st->projectile_type[i], 0, 1);
      float ang = atan2f(st->projectile_velocity_y[i], st->projectile_velocity_x[i]);
      float viewer = atan2f(py - st->projectile_y[i], px - st->projectile_x[i]);
      int rot = rotation(viewer, ang);
      int frame = type == 1 ? (int)pymod(floordiv(st->projectile_age[i], 6), 2) : 0;
      int alive = st->projectile_alive[i] != 0;
      put(&e, l, st->projectile_x[i], st->projectile_y[i], st->projectile_z[i], flight[(type * 2 + frame) * 8 + rot],
          alive, alive, type == 1 ? 0 : -1);
      e.pos++;
    }
    /* enemy projectiles in flight (14462-14510) */
    for (int s = 0; s < EP; ++s) {
      if (!used[EFLIGHT][s]) continue;
      size_t i = (size_t)l * EP + s;
      float ang = atan2f(st->enemy_projectile_velocity_y[i], st->enemy_projectile_velocity_x[i]);
      float viewer = atan2f(py - st->enemy_projectile_y[i], px - st->enemy_projectile_x[i]);
      int rot = rotation(viewer, ang);
      int frame = (int)pymod(floordiv(st->enemy_projectile_age[i], 4), 2);
      int alive = st->enemy_projectile_alive[i] != 0;
      put(&e, l, st->enemy_projectile_x[i], st->enemy_projectile_y[i], st->enemy_projectile_z[i],
          flight[(2 * 2 + frame) * 8 + rot], alive, alive, 1);
      e.pos++;
    }
    /* impacts (14512-14578, 14106-14122) */
    for (int s = 0; s < PP; ++s) {
      if (!used[PIMPACT][s]) continue;
      size_t i = (size_t)l * PP + s;
      i64 kind = st->projectile_impact_type[i];
      int safe = clampi(kind, 0, 2);
      i64 elapsed = (i64)explTotal[safe] - st->projectile_impact_tics[i];
      int sprite = explIds[safe * 5 + frame_from_ends(elapsed, &explEnds[safe * 5], 5, explCounts[safe])];
      int alive = st->projectile_impact_tics[i] > 0;
      put(&e, l, st->projectile_x[i], st->projectile_y[i], st->projectile_z[i], sprite, alive, alive, kind == 1 ? 0 : -1);
      e.pos++;
    }
    for (int s = 0; s < EP; ++s) {
      if (!used[EIMPACT][s]) continue;
      size_t i = (size_t)l * EP + s;
      i64 elapsed = (i64)explTotal[2] - st->enemy_projectile_impact_tics[i];
      int sprite = explIds[2 * 5 + frame_from_ends(elapsed, &explEnds[2 * 5], 5, explCounts[2])];
      int alive = st->enemy_projectile_impact_tics[i] > 0;
      put(&e, l, st->enemy_projectile_x[i], st->enemy_projectile_y[i], st->enemy_projectile_z[i], sprite, alive, alive, 1);
      e.pos++;
    }
    /* teleport fog (14580-14598) */
    for (int s = 0; s < E; ++s) {
      if (!used[FOG][s]) continue;
      size_t i = (size_t)l * E + s;
      i64 frame = floordiv(72 - (i64)st->teleport_fog_tics[i], 6);
      if (frame > 11) frame = 11;
      int alive = st->teleport_fog_tics[i] > 0;
      put(&e, l, st->teleport_fog_x[i], st->teleport_fog_y[i], st->teleport_fog_z[i],
          fogIds[pymod(frame, 12)], alive, alive, 1);
      e.pos++;
    }
    /* bullet puffs (14600-14629) */
    for (int s = 0; s < PF; ++s) {
      if (!used[PUFF][s]) continue;
      size_t i = (size_t)l * PF + s;
      int tics = st->hitscan_puff_tics[i];
      int frame = tics > 12 ? 0 : (tics > 8 ? 1 : (tics > 4 ? 2 : 3));
      put(&e, l, st->hitscan_puff_x[i], st->hitscan_puff_y[i], st->hitscan_puff_z[i], puffIds[frame], tics > 0,
          frame == 0, -2);
      e.pos++;
    }
    /* map items (14631-14653, 14258-14317) */
    for (int s = 0; s < I; ++s) {
      if (!used[ITEM][s]) continue;
      size_t i = (size_t)l * I + s;
      int type = itemInfo[s * 2], sprite = itemInfo[s * 2 + 1];
      i64 elapsed = (i64)st->episode_time[l] + (6 - (i64)st->item_animation_initial_tics[i]);
      int phase = (int)pymod(floordiv(elapsed, 6), 6);
      static const int bounce[6] = {-1, 0, 1, 2, 1, 0};
      if (type == 2014 && phase > 0) sprite = itemAnim[bounce[phase]];
      if (type == 2015 && phase > 0) sprite = itemAnim[3 + bounce[phase]];
      int greenBright = type == 2018 && pymod(elapsed, 13) >= 6;
      int blueBright = type == 2019 && pymod(elapsed, 12) >= 6;
      if (greenBright) sprite = itemAnim[6];
      if (blueBright) sprite = itemAnim[7];
      put(&e, l, itemPos[s * 4], itemPos[s * 4 + 1], itemPos[s * 4 + 2], sprite, st->item_available[i] != 0,
          greenBright || blueBright, -1);
      e.pos++;
    }
    /* dropped items (14655-14682) */
    for (int s = 0; s < E; ++s) {
      if (!used[DROP][s]) continue;
      size_t i = (size_t)l * E + s;
      i64 type = st->drop_type[i];
      int sprite = staticIds[12];
      if (type == 2007) sprite = staticIds[6];
      if (type == 2002) sprite = staticIds[14];
      put(&e, l, st->drop_x[i], st->drop_y[i], st->drop_z[i], sprite, type >= 0 && st->drop_spawned[i], 0, -1);
      e.pos++;
    }
    K = e.pos;

    /* lane record (engine.py:1658-1739 narrowed to 32 bits) */
    int32_t *o = lanes + (size_t)l * GD_LANE_WORDS;
    memset(o, 0, GD_LANE_WORDS * 4);
    o[GD_L_X] = fbits(px); o[GD_L_Y] = fbits(py);
    o[GD_L_ANGLE] = fbits(st->angle[l]); o[GD_L_VIEW_Z] = fbits(st->view_z[l]);
    {
      float vx = (float)st->x_fixed[l] / 65536.0f, vy = (float)st->y_fixed[l] / 65536.0f;
      i64 fx = px != vx ? (i64)rintf(px * 65536.0f) : st->x_fixed[l];
      i64 fy = py != vy ? (i64)rintf(py * 65536.0f) : st->y_fixed[l];
      o[GD_L_X_FIXED] = (int32_t)fx; o[GD_L_Y_FIXED] = (int32_t)fy;
      const float bamToRad = (float)(2.0 * M_PI / 4294967296.0);
      float visible = (float)st->angle_bam[l] * bamToRad;
      i64 pub = (i64)rintf(pyfmodf(st->angle[l], (float)(2.0 * M_PI)) / bamToRad) & 0xFFFFFFFFLL;
      i64 bam = st->angle[l] != visible ? pub : st->angle_bam[l];
      o[GD_L_ANGLE_BAM] = (int32_t)(uint32_t)(bam & 0xFFFFFFFFLL);
    }
    o[GD_L_PITCH_BAM] = (int32_t)st->pitch_bam[l];
    int flags = (st->player_dead[l] ? 1 : 0) | (st->mugshot_ouch[l] ? 2 : 0);
    if (st->render_screen_flashes) {
      int dmg = st->damage_count[l], bonus = st->bonus_count[l];
      flags |= 4 | (clampi(dmg, 0, 113) << 8) | (clampi(bonus, 0, 255) << 16);
    }
    o[GD_L_FLAGS] = flags;
    o[GD_L_EPISODE_TIME] = st->episode_time[l];
    o[GD_L_BOB_FIXED] = (int32_t)st->player_bob_fixed[l];
    o[GD_L_THINGS] = K;
    {
      i64 sel = st->selected_weapon[l];
      int slot = clampi(sel, 0, 6);
      int alt = (sel == 1 || sel == 3) && st->selected_weapon_variant[l];
      o[GD_L_WEAPON] = kSlotBaseWeapon[slot] + alt;
    }
    o[GD_L_WPN_COOLDOWN] = st->weapon_state_cooldown[l];
    o[GD_L_WPN_FIRE_COUNT] = st->weapon_fire_count[l];
    o[GD_L_WPN_READY_TICS] = st->weapon_ready_tics[l];
    o[GD_L_WPN_RAISE] = st->weapon_raise_cooldown[l];
    o[GD_L_WPN_LOWER] = st->weapon_lower_cooldown[l];
    o[GD_L_WPN_PENDING] = (int32_t)st->pending_weapon[l];
    o[GD_L_HEALTH] = fbits(st->health[l]); o[GD_L_ARMOR] = fbits(st->armor[l]);
    o[GD_L_READY_AMMO] = fbits(st->hud_ready_ammo[l]);
    for (int k = 0; k < 4; ++k) o[GD_L_AMMO0 + k] = fbits(st->hud_ammo_counts[(size_t)l * 4 + k]);
    int owned = 0;
    for (int k = 0; k < 6; ++k) owned |= (st->weapons[(size_t)l * 6 + k] != 0.0f) << k;
    o[GD_L_WEAPONS_OWNED] = owned;
    o[GD_L_FACE_INDEX] = (int32_t)st->mugshot_face_index[l];
    o[GD_L_PAIN_DIRECTION] = (int32_t)st->mugshot_pain_direction[l];
    o[GD_L_PAIN_TICS] = st->mugshot_pain_tics[l];
    o[GD_L_GRIN_TICS] = st->mugshot_grin_tics[l];
    o[GD_L_ATTACK_HELD] = st->attack_held_tics[l];
  }
  return K;
}
