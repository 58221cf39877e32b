/* Engine-shaped lane tensors -> lane records and thing records (gd_pack_state).
 * Part of gd_render.cu (one translation unit); not meant to be included elsewhere.
 *
 * Restates the actor gathering at the head of the reference's sprite pass
 * (src/gradoom/engine.py:14328-14682) with its sprite-id selection (13994-14136,
 * 14258-14317) and the view-pose selection (2122-2133, 10648-10658) as two small
 * kernels: the first marks, per actor class, the slots some lane of the batch
 * uses (the reference keeps a slot for every lane as soon as one lane uses it);
 * the second gives every lane one CTA that ranks the used slots and writes the
 * lane's records.  No host synchronisation, no allocation.
 */
#ifndef GD_STATE_CUH
#define GD_STATE_CUH

#define GD_STATE_MAX_SLOTS 2048
#define GD_STATE_THREADS 128
#define GD_STATE_CHUNK (GD_STATE_MAX_SLOTS / GD_STATE_THREADS)

/* actor classes in the order the reference concatenates them */
enum { GD_C_ENEMY, GD_C_DOLL, GD_C_CORPSE, GD_C_PFLIGHT, GD_C_EFLIGHT, GD_C_PIMPACT, GD_C_EIMPACT, GD_C_FOG, GD_C_PUFF,
       GD_C_ITEM, GD_C_DROP, GD_C_COUNT };

struct GdStateTables {
  const int32_t *walk, *attack, *pain, *deathIds, *deathCounts, *deathEnds, *xdeathIds, *xdeathCounts, *xdeathEnds;
  const int32_t *flight, *explIds, *explCounts, *explEnds, *explTotal, *fogIds, *puffIds, *staticIds, *itemInfo, *itemAnim;
  const float *starts, *itemPos;
  int deathFrames, xdeathFrames;
};

struct GdStateParams {
  gd_engine_state st;
  GdStateTables tab;
  int offset[GD_C_COUNT + 1];   /* first flat slot index of each class; [GD_C_COUNT] = total */
  int maxThings;
  unsigned *used;               /* GD_STATE_MAX_SLOTS words, zero on entry of the first kernel */
  int32_t *lanes;
  gd_thing *things;
  int *status;
};

__device__ __forceinline__ i64 gd_floordiv(i64 a, i64 b) {
  i64 q = a / b;
  return ((a % b != 0) && ((a < 0) != (b < 0))) ? q - 1 : q;
}
__device__ __forceinline__ float gd_pyfmodf(float a, float b) {
  float r = fmodf(a, b);
  return (r != 0.0f && ((b < 0) != (r < 0))) ? r + b : r;
}
/* zero-based clockwise Doom sprite rotation (src/gradoom/engine.py:13994-14009) */
__device__ __forceinline__ int gd_sprite_rotation(float viewer, float actor) {
  const float eighth = (float)(3.14159265358979323846 / 8), twoPi = (float)(2 * 3.14159265358979323846),
              quarter = (float)(3.14159265358979323846 / 4);
  float relative = gd_pyfmodf(viewer - actor + eighth, twoPi);
  return (int)gd_pymod((i64)floorf(relative / quarter), 8);
}
__device__ __forceinline__ int gd_frame_from_ends(i64 elapsed, const int32_t *ends, int frames, int count) {
  int f = 0;
  for (int k = 0; k < frames; ++k) f += elapsed >= ends[k];
  f = f < count - 1 ? f : count - 1;
  return (int)gd_pymod(f, frames);
}

/* ---- kernel 1: which slots does the batch use -------------------------------- */
__global__ void gd_state_used_kernel(const GdStateParams p) {
  const gd_engine_state &st = p.st;
  const size_t stride = (size_t)gridDim.x * blockDim.x, first = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int E = st.enemy_slots, PP = st.projectile_slots, EP = st.enemy_projectile_slots, PF = st.puff_slots,
            I = st.items;
  for (size_t i = first; i < (size_t)st.n * E; i += stride) {
    const int s = (int)(i % E);
    if (st.enemy_alive[i]) p.used[p.offset[GD_C_ENEMY] + s] = 1u;
    if (st.enemy_death_tics[i] > 0) p.used[p.offset[GD_C_CORPSE] + s] = 1u;
    if (st.teleport_fog_tics[i] > 0) p.used[p.offset[GD_C_FOG] + s] = 1u;
    if (st.drop_type[i] >= 0 && st.drop_spawned[i]) p.used[p.offset[GD_C_DROP] + s] = 1u;
  }
  for (size_t i = first; i < (size_t)st.n * PP; i += stride) {
    const int s = (int)(i % PP);
    if (st.projectile_alive[i]) p.used[p.offset[GD_C_PFLIGHT] + s] = 1u;
    if (st.projectile_impact_tics[i] > 0) p.used[p.offset[GD_C_PIMPACT] + s] = 1u;
  }
  for (size_t i = first; i < (size_t)st.n * EP; i += stride) {
    const int s = (int)(i % EP);
    if (st.enemy_projectile_alive[i]) p.used[p.offset[GD_C_EFLIGHT] + s] = 1u;
    if (st.enemy_projectile_impact_tics[i] > 0) p.used[p.offset[GD_C_EIMPACT] + s] = 1u;
  }
  for (size_t i = first; i < (size_t)st.n * PF; i += stride)
    if (st.hitscan_puff_tics[i] > 0) p.used[p.offset[GD_C_PUFF] + (int)(i % PF)] = 1u;
  for (size_t i = first; i < (size_t)st.n * I; i += stride)
    if (st.item_available[i]) p.used[p.offset[GD_C_ITEM] + (int)(i % I)] = 1u;
  /* the voodoo dolls at the unused player starts are always listed */
  for (size_t i = first; i < (size_t)(p.offset[GD_C_DOLL + 1] - p.offset[GD_C_DOLL]); i += stride)
    p.used[p.offset[GD_C_DOLL] + i] = 1u;
}

/* ---- kernel 2: one CTA per lane writes its records ---------------------------- */
__device__ void gd_state_record(const GdStateParams &p, int l, int cls, int s, gd_thing &out) {
  const gd_engine_state &st = p.st;
  const GdStateTables &t = p.tab;
  const float px = st.x[l], py = st.y[l];
  float x = 0, y = 0, z = 0;
  int sprite = 0, style = -1;
  bool alive = false, bright = false;
  switch (cls) {
    case GD_C_ENEMY: {   /* engine.py:14330-14343, 14011-14077, 14124-14136 */
      const size_t i = (size_t)l * st.enemy_slots + s;
      const int type = (int)gd_clamp(st.enemy_type[i], 0, 5);
      const int kWalk[6] = {8, 6, 4, 6, 4, 6}, kIdle[6] = {10, 10, 8, 10, 10, 10}, kRecovery[6] = {16, 20, 4, 4, 8, 8};
      x = st.enemy_x[i]; y = st.enemy_y[i]; z = st.enemy_z[i];
      const float viewer = atan2f(py - y, px - x);
      const int rot = gd_sprite_rotation(viewer, st.enemy_angle[i]);
      const i64 tics = st.enemy_animation_tics[i];
      int walkFrame = (int)gd_pymod(gd_floordiv(tics, kWalk[type]), 4);
      int idleFrame = (int)gd_pymod(gd_floordiv(tics, kIdle[type]), 2);
      if (type == 2) idleFrame = 0;
      if (st.enemy_target_slot[i] < -1) walkFrame = idleFrame;
      const int phase = st.enemy_attack_phase[i], cooldown = st.enemy_cooldown[i];
      const int recovering = cooldown > (kRecovery[type] / 2);
      int attackFrame = 0;
      if (type == 0 || type == 1) attackFrame = phase == 2 ? recovering : 0;
      if ((type == 4 || type == 5) && phase == 1) attackFrame = cooldown <= 8;
      if ((type == 4 || type == 5) && phase == 2) attackFrame = 2;
      if (type == 3 && (phase == 4 || phase == 2)) attackFrame = 1;
      if (type == 3 && phase == 3) attackFrame = 2;
      sprite = phase > 0 ? t.attack[(type * 4 + attackFrame) * 8 + rot] : t.walk[(type * 4 + walkFrame) * 8 + rot];
      if (st.enemy_pain_tics[i] > 0) sprite = t.pain[type * 8 + rot];
      bright = (type == 1 && phase == 2 && recovering) || (type == 3 && (phase == 2 || phase == 3));
      alive = st.enemy_alive[i] != 0;
      break;
    }
    case GD_C_DOLL: {    /* 14345-14381 */
      const float *sp = &t.starts[s * 4];
      x = sp[0]; y = sp[1]; z = sp[3];
      const int rot = gd_sprite_rotation(atan2f(py - y, px - x), sp[2]);
      sprite = t.walk[(2 * 4 + 0) * 8 + rot];
      alive = !st.player_dead[l];
      break;
    }
    case GD_C_CORPSE: {  /* 14383-14410, 14079-14104 */
      const size_t i = (size_t)l * st.enemy_slots + s;
      const int type = (int)gd_clamp(st.enemy_death_type[i], 0, 5);
      const i64 elapsed = st.enemy_death_elapsed[i];
      x = st.enemy_x[i]; y = st.enemy_y[i]; z = st.enemy_z[i];
      sprite = st.enemy_death_extreme[i]
                   ? t.xdeathIds[type * t.xdeathFrames +
                                 gd_frame_from_ends(elapsed, &t.xdeathEnds[type * t.xdeathFrames], t.xdeathFrames, t.xdeathCounts[type])]
                   : t.deathIds[type * t.deathFrames +
                                gd_frame_from_ends(elapsed, &t.deathEnds[type * t.deathFrames], t.deathFrames, t.deathCounts[type])];
      alive = st.enemy_death_tics[i] > 0;
      break;
    }
    case GD_C_PFLIGHT: { /* 14412-14460 */
      const size_t i = (size_t)l * st.projectile_slots + s;
      const int type = (int)gd_clamp(st.projectile_type[i], 0, 1);
      x = st.projectile_x[i]; y = st.projectile_y[i]; z = st.projectile_z[i];
      const float ang = atan2f(st.projectile_velocity_y[i], st.projectile_velocity_x[i]);
      const int rot = gd_sprite_rotation(atan2f(py - y, px - x), ang);
      const int frame = type == 1 ? (int)gd_pymod(gd_floordiv(st.projectile_age[i], 6), 2) : 0;
      sprite = t.flight[(type * 2 + frame) * 8 + rot];
      alive = bright = st.projectile_alive[i] != 0;
      style = type == 1 ? 0 : -1;
      break;
    }
    case GD_C_EFLIGHT: { /* 14462-14510 */
      const size_t i = (size_t)l * st.enemy_projectile_slots + s;
      x = st.enemy_projectile_x[i]; y = st.enemy_projectile_y[i]; z = st.enemy_projectile_z[i];
      const float ang = atan2f(st.enemy_projectile_velocity_y[i], st.enemy_projectile_velocity_x[i]);
      const int rot = gd_sprite_rotation(atan2f(py - y, px - x), ang);
      const int frame = (int)gd_pymod(gd_floordiv(st.enemy_projectile_age[i], 4), 2);
      sprite = t.flight[(2 * 2 + frame) * 8 + rot];
      alive = bright = st.enemy_projectile_alive[i] != 0;
      style = 1;
      break;
    }
    case GD_C_PIMPACT: { /* 14512-14545, 14106-14122 */
      const size_t i = (size_t)l * st.projectile_slots + s;
      const i64 kind = st.projectile_impact_type[i];
      const int safe = (int)gd_clamp(kind, 0, 2);
      const i64 elapsed = (i64)t.explTotal[safe] - st.projectile_impact_tics[i];
      x = st.projectile_x[i]; y = st.projectile_y[i]; z = st.projectile_z[i];
      sprite = t.explIds[safe * 5 + gd_frame_from_ends(elapsed, &t.explEnds[safe * 5], 5, t.explCounts[safe])];
      alive = bright = st.projectile_impact_tics[i] > 0;
      style = kind == 1 ? 0 : -1;
      break;
    }
    case GD_C_EIMPACT: { /* 14547-14578 */
      const size_t i = (size_t)l * st.enemy_projectile_slots + s;
      const i64 elapsed = (i64)t.explTotal[2] - st.enemy_projectile_impact_tics[i];
      x = st.enemy_projectile_x[i]; y = st.enemy_projectile_y[i]; z = st.enemy_projectile_z[i];
      sprite = t.explIds[2 * 5 + gd_frame_from_ends(elapsed, &t.explEnds[2 * 5], 5, t.explCounts[2])];
      alive = bright = st.enemy_projectile_impact_tics[i] > 0;
      style = 1;
      break;
    }
    case GD_C_FOG: {     /* 14580-14598 */
      const size_t i = (size_t)l * st.enemy_slots + s;
      i64 frame = gd_floordiv(72 - (i64)st.teleport_fog_tics[i], 6);
      if (frame > 11) frame = 11;
      x = st.teleport_fog_x[i]; y = st.teleport_fog_y[i]; z = st.teleport_fog_z[i];
      sprite = t.fogIds[gd_pymod(frame, 12)];
      alive = bright = st.teleport_fog_tics[i] > 0;
      style = 1;
      break;
    }
    case GD_C_PUFF: {    /* 14600-14629 */
      const size_t i = (size_t)l * st.puff_slots + s;
      const int tics = st.hitscan_puff_tics[i];
      const int frame = tics > 12 ? 0 : (tics > 8 ? 1 : (tics > 4 ? 2 : 3));
      x = st.hitscan_puff_x[i]; y = st.hitscan_puff_y[i]; z = st.hitscan_puff_z[i];
      sprite = t.puffIds[frame];
      alive = tics > 0; bright = frame == 0; style = -2;
      break;
    }
    case GD_C_ITEM: {    /* 14631-14653, 14258-14317 */
      const size_t i = (size_t)l * st.items + s;
      const int type = t.itemInfo[s * 2];
      sprite = t.itemInfo[s * 2 + 1];
      const i64 elapsed = (i64)st.episode_time[l] + (6 - (i64)st.item_animation_initial_tics[i]);
      const int phase = (int)gd_pymod(gd_floordiv(elapsed, 6), 6);
      const int bounce = phase <= 3 ? phase - 1 : 5 - phase;       /* frames A B C D C B */
      if (type == 2014 && phase > 0) sprite = t.itemAnim[bounce];
      if (type == 2015 && phase > 0) sprite = t.itemAnim[3 + bounce];
      const bool green = type == 2018 && gd_pymod(elapsed, 13) >= 6, blue = type == 2019 && gd_pymod(elapsed, 12) >= 6;
      if (green) sprite = t.itemAnim[6];
      if (blue) sprite = t.itemAnim[7];
      x = t.itemPos[s * 4]; y = t.itemPos[s * 4 + 1]; z = t.itemPos[s * 4 + 2];
      alive = st.item_available[i] != 0;
      bright = green || blue;
      break;
    }
    default: {           /* dropped items, 14655-14682 */
      const size_t i = (size_t)l * st.enemy_slots + s;
      const i64 type = st.drop_type[i];
      sprite = t.staticIds[12];
      if (type == 2007) sprite = t.staticIds[6];
      if (type == 2002) sprite = t.staticIds[14];
      x = st.drop_x[i]; y = st.drop_y[i]; z = st.drop_z[i];
      alive = type >= 0 && st.drop_spawned[i];
      break;
    }
  }
  out.x = x; out.y = y; out.z = z;
  out.sprite = (uint16_t)sprite;
  out.flags = (uint8_t)((alive ? GD_THING_ALIVE : 0) | (bright ? GD_THING_BRIGHT : 0));
  out.style = (int8_t)style;
}

__device__ void gd_state_lane_record(const GdStateParams &p, int l, int K) {
  const gd_engine_state &st = p.st;
  int32_t *o = p.lanes + (size_t)l * GD_LANE_WORDS;
  const float px = st.x[l], py = st.y[l], angle = st.angle[l];
  o[GD_L_X] = __float_as_int(px); o[GD_L_Y] = __float_as_int(py);
  o[GD_L_ANGLE] = __float_as_int(angle); o[GD_L_VIEW_Z] = __float_as_int(st.view_z[l]);
  /* a public coordinate or angle that was changed behind the retained fixed-point
   * value wins (engine.py:2122-2133, 10648-10658) */
  const i64 xf = st.x_fixed[l], yf = st.y_fixed[l], bamRetained = st.angle_bam[l];
  const float vx = (float)xf / 65536.0f, vy = (float)yf / 65536.0f;
  o[GD_L_X_FIXED] = (int32_t)(px != vx ? (i64)rintf(px * 65536.0f) : xf);
  o[GD_L_Y_FIXED] = (int32_t)(py != vy ? (i64)rintf(py * 65536.0f) : yf);
  const float bamToRad = (float)(2.0 * 3.14159265358979323846 / 4294967296.0);
  const float visible = (float)bamRetained * bamToRad;
  const i64 pub = (i64)rintf(gd_pyfmodf(angle, (float)(2.0 * 3.14159265358979323846)) / bamToRad) & 0xFFFFFFFFLL;
  o[GD_L_ANGLE_BAM] = (int32_t)(uint32_t)((angle != visible ? pub : bamRetained) & 0xFFFFFFFFLL);
  o[GD_L_PITCH_BAM] = (int32_t)st.pitch_bam[l];
  int flags = (st.player_dead[l] ? 1 : 0) | (st.mugshot_ouch[l] ? 2 : 0);
  if (st.render_screen_flashes)
    flags |= 4 | ((int)gd_clamp(st.damage_count[l], 0, 113) << 8) | ((int)gd_clamp(st.bonus_count[l], 0, 255) << 16);
  o[GD_L_FLAGS] = flags;
  o[GD_L_EPISODE_TIME] = st.episode_time[l];
  o[GD_L_BOB_FIXED] = (int32_t)st.player_bob_fixed[l];
  o[GD_L_THINGS] = K;
  {
    const i64 sel = st.selected_weapon[l];
    const int slot = (int)gd_clamp(sel, 0, 6);
    const int base = slot < 2 ? 0 : (slot == 2 ? 2 : (slot == 3 ? 3 : slot + 1));     /* 0 0 2 3 5 6 7 */
    o[GD_L_WEAPON] = base + (((sel == 1 || sel == 3) && st.selected_weapon_variant[l]) ? 1 : 0);
  }
  o[GD_L_WPN_COOLDOWN] = st.weapon_state_cooldown[l];
  o[GD_L_WPN_FIRE_COUNT] = st.weapon_fire_count[l];
  o[GD_L_WPN_READY_TICS] = st.weapon_ready_tics[l];
  o[GD_L_WPN_RAISE] = st.weapon_raise_cooldown[l];
  o[GD_L_WPN_LOWER] = st.weapon_lower_cooldown[l];
  o[GD_L_WPN_PENDING] = (int32_t)st.pending_weapon[l];
  o[GD_L_HEALTH] = __float_as_int(st.health[l]); o[GD_L_ARMOR] = __float_as_int(st.armor[l]);
  o[GD_L_READY_AMMO] = __float_as_int(st.hud_ready_ammo[l]);
  for (int k = 0; k < 4; ++k) o[GD_L_AMMO0 + k] = __float_as_int(st.hud_ammo_counts[(size_t)l * 4 + k]);
  int owned = 0;
  for (int k = 0; k < 6; ++k) owned |= (st.weapons[(size_t)l * 6 + k] != 0.0f) << k;
  o[GD_L_WEAPONS_OWNED] = owned;
  o[GD_L_FACE_INDEX] = (int32_t)st.mugshot_face_index[l];
  o[GD_L_PAIN_DIRECTION] = (int32_t)st.mugshot_pain_direction[l];
  o[GD_L_PAIN_TICS] = st.mugshot_pain_tics[l];
  o[GD_L_GRIN_TICS] = st.mugshot_grin_tics[l];
  o[GD_L_ATTACK_HELD] = st.attack_held_tics[l];
}

__global__ void __launch_bounds__(GD_STATE_THREADS) gd_state_emit_kernel(const GdStateParams p) {
  __shared__ unsigned short rank[GD_STATE_MAX_SLOTS];
  __shared__ int chunkCount[GD_STATE_THREADS + 1];
  const int tid = threadIdx.x, l = blockIdx.x, total = p.offset[GD_C_COUNT];
  /* rank of every used slot: a count per thread chunk, a serial scan of the 128
   * counts, then the ranks inside each chunk */
  const int g0 = tid * GD_STATE_CHUNK;
  int mine = 0;
  for (int k = 0; k < GD_STATE_CHUNK; ++k) {
    const int g = g0 + k;
    mine += (g < total && p.used[g]) ? 1 : 0;
  }
  chunkCount[tid + 1] = mine;
  __syncthreads();
  if (tid == 0) {
    chunkCount[0] = 0;
    for (int k = 1; k <= GD_STATE_THREADS; ++k) chunkCount[k] += chunkCount[k - 1];
  }
  __syncthreads();
  const int K = chunkCount[GD_STATE_THREADS];
  int pos = chunkCount[tid];
  for (int k = 0; k < GD_STATE_CHUNK; ++k) {
    const int g = g0 + k;
    const bool on = g < total && p.used[g];
    rank[g] = (unsigned short)(on ? pos : 0xFFFF);
    pos += on ? 1 : 0;
  }
  __syncthreads();
  const int stride = p.maxThings > 0 ? p.maxThings : 1;
  for (int g = tid; g < total; g += GD_STATE_THREADS) {
    const int at = rank[g];
    if (at == 0xFFFF || at >= p.maxThings) continue;
    int cls = 0;
    while (g >= p.offset[cls + 1]) ++cls;
    gd_thing rec;
    gd_state_record(p, l, cls, g - p.offset[cls], rec);
    p.things[(size_t)l * stride + at] = rec;
  }
  if (tid == 0) {
    gd_state_lane_record(p, l, K);
    if (K > p.maxThings && l == 0) atomicOr(p.status, GD_STATUS_THINGS_OVERFLOW);
  }
}

#endif
