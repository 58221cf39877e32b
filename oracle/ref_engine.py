"""Bridge to the upstream Torch engine (TEST INFRASTRUCTURE, never on the product path).

Two users: ``tests/golden/make_golden.py`` runs the upstream CPU renderer on seeded
synthetic scenes to record the golden fixtures, and the reference arm of ``bench.py``
times the upstream engine on the host cores.  The upstream package is pure Python;
``install()`` puts an unmodified copy of its ``src/gradoom`` package under
``oracle/_ref/`` (git-ignored, so it never enters the history, but it travels with the
working tree to the machine that runs the benchmark), the way ``pip install --target``
would.  ``load()`` imports the engine module from there, or from the directory named by
``GRADOOM_REFERENCE_SRC``.
"""

from __future__ import annotations

import importlib
import os
import sys
import types

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
INSTALLED = os.path.join(HERE, "_ref", "gradoom")


def install(upstream_checkout: str) -> str | None:
    """Copy the upstream package, unmodified, to ``oracle/_ref/gradoom``.  Returns the
    directory, or None when the checkout is not on this machine."""

    import shutil

    src = os.path.join(upstream_checkout, "src", "gradoom")
    if not os.path.isdir(src):
        return INSTALLED if os.path.isdir(INSTALLED) else None
    if os.path.isdir(INSTALLED):
        shutil.rmtree(INSTALLED)
    shutil.copytree(src, INSTALLED, ignore=shutil.ignore_patterns("__pycache__", "*.pyc"))
    return INSTALLED


def source_dir() -> str | None:
    env = os.environ.get("GRADOOM_REFERENCE_SRC", "")   # <upstream checkout>/src/gradoom
    if os.path.isdir(env):
        return env
    return INSTALLED if os.path.isdir(INSTALLED) else None


def load_reference():
    """Import ``gradoom.engine`` without running the package ``__init__``.

    The package ``__init__`` imports gymnasium, which is not installed; the
    engine module itself only needs numpy and torch.
    """

    src = source_dir()
    if src is None:
        raise SystemExit("the upstream package is neither installed under oracle/_ref nor named by "
                         "GRADOOM_REFERENCE_SRC (<upstream checkout>/src/gradoom)")
    if "gradoom" not in sys.modules:
        pkg = types.ModuleType("gradoom")
        pkg.__path__ = [src]
        sys.modules["gradoom"] = pkg
    engine = importlib.import_module("gradoom.engine")
    scenario = importlib.import_module("gradoom.scenario")
    actions = importlib.import_module("gradoom.actions")
    return engine, scenario, actions


def scene_to_compiled(scene, scenario_module):
    """Convert this repository's Scene into the upstream CompiledScenario."""

    walls = scene.walls.astype(np.float32)
    one_sided = scene.wall_sectors[:, 1] < 0
    verts = np.unique(walls.reshape(-1, 2), axis=0).astype(np.float32)
    gray = (
        scene.playpal[:, 0].astype(np.int32) * 77
        + scene.playpal[:, 1].astype(np.int32) * 150
        + scene.playpal[:, 2].astype(np.int32) * 29
        + 128
    ) >> 8
    gray = gray.astype(np.uint8)
    W = len(walls)
    middle = scene.side_textures[:, 0, 0]
    items = scene.meta.get("items")
    decals = scene.meta.get("decals") or {}
    fragments = fragment_mask = None
    split = scene.meta.get("fragments")
    if split:
        most = max(len(pieces) for pieces in split.values())
        fragments = np.zeros((W, most, 4), dtype=np.int64)
        fragment_mask = np.zeros((W, most), dtype=np.bool_)
        fragments[:, 0] = np.rint(walls.astype(np.float64) * 65536.0).astype(np.int64)
        fragment_mask[:, 0] = True
        for line, pieces in split.items():
            fragments[line, : len(pieces)] = pieces
            fragment_mask[line, : len(pieces)] = True
    return scenario_module.CompiledScenario(
        wall_projection_fragments_fixed=fragments,
        wall_projection_fragment_mask=fragment_mask,
        bullet_decal_atlas=decals.get("atlas"),
        bullet_decal_heights=decals.get("heights"),
        bullet_decal_left_offsets=decals.get("left"),
        bullet_decal_top_offsets=decals.get("top"),
        bullet_decal_opacity_lut=decals.get("opacity_lut"),
        bullet_decal_black_lut=decals.get("black_lut"),
        scenario_sha256="0" * 64,
        iwad_sha256="1" * 64,
        namespace="zdoom",
        vertices=verts,
        wall_segments=walls,
        blocking_segments=walls[one_sided].copy(),
        blocking_wall_indices=np.flatnonzero(one_sided).astype(np.int32),
        wall_texture_ids=np.where(middle >= 0, middle, 0).astype(np.int32),
        wall_texture_offsets=np.zeros((W, 2), dtype=np.float32),
        wall_side_texture_ids=scene.side_textures.astype(np.int32),
        wall_side_texture_offsets=scene.side_offsets.astype(np.float32),
        wall_sectors=scene.wall_sectors.astype(np.int32),
        sector_edge_mask=scene.sector_edge_mask,
        sector_heights=scene.sector_heights.astype(np.float32),
        sector_lights=scene.sector_lights.astype(np.int16),
        sector_floor_texture_ids=scene.sector_floor_tex.astype(np.int32),
        sector_ceiling_texture_ids=scene.sector_ceil_tex.astype(np.int32),
        player_starts=scene.player_starts.astype(np.float32),
        item_spawns=np.empty((0, 3), dtype=np.float32) if items is None else items["spawns"].astype(np.float32),
        item_types=np.empty((0,), dtype=np.int32) if items is None else items["types"].astype(np.int32),
        raw_item_animation_sprite_ids=None if items is None else items["anim_ids"].astype(np.int32),
        playpal=scene.playpal,
        texture_names=tuple(f"T{i}" for i in range(len(scene.tex_atlas))),
        texture_atlas=gray[scene.tex_atlas],
        texture_widths=scene.tex_widths,
        texture_heights=scene.tex_heights,
        sprite_names=tuple(f"S{i}" for i in range(26)),
        sprite_atlas=np.full((26, 1, 1), 224, dtype=np.uint8),
        sprite_opaque=np.ones((26, 1, 1), dtype=np.bool_),
        sprite_widths=np.ones(26, dtype=np.int32),
        sprite_heights=np.ones(26, dtype=np.int32),
        sprite_left_offsets=np.zeros(26, dtype=np.int32),
        sprite_top_offsets=np.full(26, 42, dtype=np.int32),
        weapon_sprite_names=tuple(f"W{i}" for i in range(8)),
        weapon_screen_values=np.zeros((8, 84, 84), dtype=np.float32),
        weapon_screen_alpha=np.zeros((8, 84, 84), dtype=np.float32),
        texture_index_atlas=scene.tex_atlas,
        colormap=scene.colormap,
        raw_sprite_names=tuple(f"R{i}" for i in range(len(scene.spr_atlas))),
        raw_sprite_atlas=scene.spr_atlas,
        raw_sprite_opaque=scene.spr_opaque,
        raw_sprite_widths=scene.spr_widths,
        raw_sprite_heights=scene.spr_heights,
        raw_sprite_left_offsets=scene.spr_left,
        raw_sprite_top_offsets=scene.spr_top,
        enemy_walk_sprite_ids=scene.enemy_walk_ids,
        enemy_attack_sprite_ids=scene.enemy_attack_ids,
        enemy_death_sprite_ids=scene.enemy_death_ids,
        enemy_death_frame_counts=scene.enemy_death_counts,
        enemy_death_frame_durations=scene.enemy_death_durations,
        enemy_xdeath_sprite_ids=scene.enemy_xdeath_ids,
        enemy_xdeath_frame_counts=scene.enemy_xdeath_counts,
        enemy_xdeath_frame_durations=scene.enemy_xdeath_durations,
        enemy_pain_sprite_ids=scene.enemy_pain_ids,
        raw_projectile_flight_sprite_ids=scene.proj_flight_ids,
        raw_projectile_explosion_sprite_ids=scene.proj_explosion_ids,
        raw_teleport_fog_sprite_ids=scene.fog_ids,
        projectile_explosion_frame_counts=scene.proj_explosion_counts,
        projectile_explosion_frame_durations=scene.proj_explosion_durations,
        projectile_additive_luts=scene.additive_luts,
        sprite_translucent_lut=scene.translucent_lut,
        raw_bullet_puff_sprite_ids=scene.puff_ids,
        raw_static_sprite_ids=scene.static_ids,
        native_weapon_patch_atlas=scene.wpn_atlas if scene.wpn_widths.max() > 0 else None,
        native_weapon_patch_opaque=scene.wpn_opaque if scene.wpn_widths.max() > 0 else None,
        native_weapon_patch_widths=scene.wpn_widths if scene.wpn_widths.max() > 0 else None,
        native_weapon_patch_heights=scene.wpn_heights if scene.wpn_widths.max() > 0 else None,
        native_weapon_patch_left_offsets=scene.wpn_left if scene.wpn_widths.max() > 0 else None,
        native_weapon_patch_top_offsets=scene.wpn_top if scene.wpn_widths.max() > 0 else None,
        native_weapon_frame_ids=scene.wpn_frame_ids,
        native_weapon_flash_ids=scene.wpn_flash_ids,
        native_weapon_flash_lights=scene.wpn_flash_lights,
        hud_patch_names=tuple(f"H{i}" for i in range(len(scene.hud_atlas))),
        hud_patch_atlas=scene.hud_atlas,
        hud_patch_opaque=scene.hud_opaque,
        hud_patch_widths=scene.hud_widths,
        hud_patch_heights=scene.hud_heights,
        hud_patch_left_offsets=scene.hud_left,
        hud_patch_top_offsets=scene.hud_top,
    )
