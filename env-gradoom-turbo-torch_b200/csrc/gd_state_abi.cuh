/* C ABI of gd_pack_state (declared in include/gradoom_b200.h).
 * Part of gd_render.cu (one translation unit); not meant to be included elsewhere. */
#ifndef GD_STATE_ABI_CUH
#define GD_STATE_ABI_CUH

extern "C" size_t gd_pack_state_scratch_bytes(void) { return (size_t)GD_STATE_MAX_SLOTS * sizeof(unsigned); }

extern "C" int gd_pack_state(const gd_renderer *r, const gd_engine_state *state, int32_t *lanes, void *things,
                             void *flags_scratch, size_t flags_scratch_bytes, int *status, void *stream) {
  if (!r || !state || !lanes || !flags_scratch || !status) return GD_ERR_NULL;
  if (r->maxThings > 0 && !things) return GD_ERR_NULL;
  const gd_engine_state &st = *state;
  if (st.n < 0 || st.enemy_slots < 0 || st.projectile_slots < 0 || st.enemy_projectile_slots < 0 || st.puff_slots < 0 ||
      st.items < 0)
    return GD_ERR_SIZE;
  if (st.n == 0) return GD_OK;
  if (st.items != r->header[GD_H_ITEMS]) return GD_ERR_SIZE;
  if (flags_scratch_bytes < gd_pack_state_scratch_bytes()) return GD_ERR_SCRATCH;
  if (((uintptr_t)lanes | (uintptr_t)things | (uintptr_t)flags_scratch) & 15) return GD_ERR_ALIGN;
  /* every tensor of a class that has slots must be there */
  const void *player[] = {st.x, st.y, st.angle, st.view_z, st.health, st.armor, st.hud_ready_ammo, st.x_fixed, st.y_fixed,
                          st.angle_bam, st.pitch_bam, st.player_bob_fixed, st.selected_weapon, st.pending_weapon,
                          st.mugshot_face_index, st.mugshot_pain_direction, st.episode_time, st.weapon_state_cooldown,
                          st.weapon_fire_count, st.weapon_ready_tics, st.weapon_raise_cooldown, st.weapon_lower_cooldown,
                          st.mugshot_pain_tics, st.mugshot_grin_tics, st.attack_held_tics, st.player_dead,
                          st.selected_weapon_variant, st.mugshot_ouch, st.hud_ammo_counts, st.weapons};
  for (const void *q : player) if (!q) return GD_ERR_NULL;
  if (st.render_screen_flashes && (!st.damage_count || !st.bonus_count)) return GD_ERR_NULL;
  if (st.enemy_slots > 0) {
    const void *need[] = {st.enemy_x, st.enemy_y, st.enemy_z, st.enemy_angle, st.enemy_type, st.enemy_target_slot,
                          st.enemy_death_type, st.enemy_animation_tics, st.enemy_attack_phase, st.enemy_cooldown,
                          st.enemy_pain_tics, st.enemy_death_tics, st.enemy_death_elapsed, st.enemy_alive,
                          st.enemy_death_extreme, st.teleport_fog_x, st.teleport_fog_y, st.teleport_fog_z,
                          st.teleport_fog_tics, st.drop_x, st.drop_y, st.drop_z, st.drop_type, st.drop_spawned};
    for (const void *q : need) if (!q) return GD_ERR_NULL;
  }
  if (st.projectile_slots > 0) {
    const void *need[] = {st.projectile_x, st.projectile_y, st.projectile_z, st.projectile_velocity_x,
                          st.projectile_velocity_y, st.projectile_type, st.projectile_impact_type, st.projectile_age,
                          st.projectile_impact_tics, st.projectile_alive};
    for (const void *q : need) if (!q) return GD_ERR_NULL;
  }
  if (st.enemy_projectile_slots > 0) {
    const void *need[] = {st.enemy_projectile_x, st.enemy_projectile_y, st.enemy_projectile_z,
                          st.enemy_projectile_velocity_x, st.enemy_projectile_velocity_y, st.enemy_projectile_age,
                          st.enemy_projectile_impact_tics, st.enemy_projectile_alive};
    for (const void *q : need) if (!q) return GD_ERR_NULL;
  }
  if (st.puff_slots > 0 && (!st.hitscan_puff_x || !st.hitscan_puff_y || !st.hitscan_puff_z || !st.hitscan_puff_tics))
    return GD_ERR_NULL;
  if (st.items > 0 && (!st.item_available || !st.item_animation_initial_tics)) return GD_ERR_NULL;
  int current = -1;
  if (cudaGetDevice(&current) != cudaSuccess) return GD_ERR_CUDA;
  if (current != r->device) return GD_ERR_DEVICE;

  GdStateParams p;
  p.st = st;
  const int32_t *h = r->header;
  const uint8_t *d = (const uint8_t *)r->blobDev;
#define SECP(type, name) (const type *)gd_section(d, h, name)
  GdStateTables &t = p.tab;
  t.walk = SECP(int32_t, GD_S_ENEMY_WALK); t.attack = SECP(int32_t, GD_S_ENEMY_ATTACK); t.pain = SECP(int32_t, GD_S_ENEMY_PAIN);
  t.deathIds = SECP(int32_t, GD_S_DEATH_IDS); t.deathCounts = SECP(int32_t, GD_S_DEATH_COUNTS);
  t.deathEnds = SECP(int32_t, GD_S_DEATH_ENDS); t.xdeathIds = SECP(int32_t, GD_S_XDEATH_IDS);
  t.xdeathCounts = SECP(int32_t, GD_S_XDEATH_COUNTS); t.xdeathEnds = SECP(int32_t, GD_S_XDEATH_ENDS);
  t.flight = SECP(int32_t, GD_S_PROJ_FLIGHT); t.explIds = SECP(int32_t, GD_S_PROJ_EXPL_IDS);
  t.explCounts = SECP(int32_t, GD_S_PROJ_EXPL_COUNTS); t.explEnds = SECP(int32_t, GD_S_PROJ_EXPL_ENDS);
  t.explTotal = SECP(int32_t, GD_S_PROJ_EXPL_TOTAL); t.fogIds = SECP(int32_t, GD_S_FOG_IDS);
  t.puffIds = SECP(int32_t, GD_S_PUFF_IDS); t.staticIds = SECP(int32_t, GD_S_STATIC_IDS);
  t.itemInfo = SECP(int32_t, GD_S_ITEM_INFO); t.itemAnim = SECP(int32_t, GD_S_ITEM_ANIM);
  t.starts = SECP(float, GD_S_STARTS); t.itemPos = SECP(float, GD_S_ITEM_POS);
#undef SECP
  t.deathFrames = h[GD_H_DEATH_FRAMES]; t.xdeathFrames = h[GD_H_XDEATH_FRAMES];
  const int dolls = h[GD_H_STARTS] > 0 ? h[GD_H_STARTS] - 1 : 0;
  const int sizes[GD_C_COUNT] = {st.enemy_slots, dolls, st.enemy_slots, st.projectile_slots, st.enemy_projectile_slots,
                                 st.projectile_slots, st.enemy_projectile_slots, st.enemy_slots, st.puff_slots, st.items,
                                 st.enemy_slots};
  p.offset[0] = 0;
  for (int c = 0; c < GD_C_COUNT; ++c) p.offset[c + 1] = p.offset[c] + sizes[c];
  if (p.offset[GD_C_COUNT] > GD_STATE_MAX_SLOTS) return GD_ERR_SIZE;
  p.maxThings = r->maxThings;
  p.used = (unsigned *)flags_scratch;
  p.lanes = lanes;
  p.things = (gd_thing *)things;
  p.status = status;
  cudaStream_t s = (cudaStream_t)stream;
  if (cudaMemsetAsync(flags_scratch, 0, gd_pack_state_scratch_bytes(), s) != cudaSuccess) return GD_ERR_CUDA;
  const size_t widest = (size_t)st.n * (size_t)(st.enemy_slots > st.enemy_projectile_slots ? st.enemy_slots : st.enemy_projectile_slots);
  int blocks = (int)((widest + 255) / 256);
  if (blocks < 1) blocks = 1;
  if (blocks > 1184) blocks = 1184;   /* eight blocks of 256 threads per SM of a 148-SM part */
  gd_state_used_kernel<<<blocks, 256, 0, s>>>(p);
  gd_state_emit_kernel<<<st.n, GD_STATE_THREADS, 0, s>>>(p);
  return cudaGetLastError() == cudaSuccess ? GD_OK : GD_ERR_CUDA;
}

#endif
