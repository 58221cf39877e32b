"""Record what the upstream WAD / UDMF / texture pipeline makes of the synthetic WAD pair.

Run once on a machine that has the upstream sources:

    GRADOOM_REFERENCE_SRC=<upstream checkout>/src/gradoom python tests/golden/make_wad_golden.py

The pair is built, byte by byte, by ``tests/wadgen.py`` from a seed, written to a temporary
directory and compiled by the upstream ``compile_deathmatch_scenario`` (scenario.py:457-1064, with
the pin on the certified map switched off and the bundled bullet-chip resource, which is under
another licence and not part of either WAD, replaced by an empty atlas).  The fixture
``golden_wad.json`` holds the digests of the two WAD files and, for every table of the compiled
scenario, its dtype, shape and SHA-256; ``tests/test_wad.py`` compiles the same bytes with this
package's reader and compares.
"""

from __future__ import annotations

import hashlib
import json
import os
import sys
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))
sys.path.insert(0, os.path.join(ROOT, "oracle"))

from __graft_entry__ import load_package  # noqa: E402

load_package()
import ref_engine  # noqa: E402
import wadgen  # noqa: E402
from gradoom_b200 import scene as gdscene, wad as gdwad  # noqa: E402

FIELDS = (
    "vertices wall_segments blocking_segments blocking_wall_indices wall_texture_ids wall_texture_offsets "
    "wall_side_texture_ids wall_side_texture_offsets wall_sectors sector_edge_mask sector_heights sector_lights "
    "sector_floor_texture_ids sector_ceiling_texture_ids player_starts item_spawns item_types playpal colormap "
    "texture_index_atlas texture_widths texture_heights raw_sprite_atlas raw_sprite_opaque raw_sprite_widths "
    "raw_sprite_heights raw_sprite_left_offsets raw_sprite_top_offsets enemy_walk_sprite_ids enemy_attack_sprite_ids "
    "enemy_pain_sprite_ids enemy_death_sprite_ids enemy_death_frame_counts enemy_death_frame_durations "
    "enemy_xdeath_sprite_ids enemy_xdeath_frame_counts enemy_xdeath_frame_durations raw_projectile_flight_sprite_ids "
    "raw_projectile_explosion_sprite_ids projectile_explosion_frame_counts projectile_explosion_frame_durations "
    "raw_teleport_fog_sprite_ids raw_bullet_puff_sprite_ids raw_static_sprite_ids raw_item_animation_sprite_ids "
    "projectile_additive_luts sprite_translucent_lut bullet_decal_opacity_lut bullet_decal_black_lut "
    "native_weapon_patch_atlas native_weapon_patch_opaque native_weapon_patch_widths native_weapon_patch_heights "
    "native_weapon_patch_left_offsets native_weapon_patch_top_offsets native_weapon_frame_ids native_weapon_flash_ids "
    "native_weapon_flash_lights hud_patch_atlas hud_patch_opaque hud_patch_widths hud_patch_heights "
    "hud_patch_left_offsets hud_patch_top_offsets"
).split()
NAMES = ("namespace", "texture_names", "raw_sprite_names", "hud_patch_names")


def digest(value) -> dict:
    a = np.ascontiguousarray(value)
    return {"dtype": str(a.dtype), "shape": list(a.shape), "sha256": hashlib.sha256(a.tobytes()).hexdigest()}


def summarize(cs) -> dict:
    out = {name: digest(getattr(cs, name)) for name in FIELDS}
    for name in NAMES:
        value = getattr(cs, name)
        out[name] = value if isinstance(value, str) else list(value)
    return out


def main():
    _eng, scn, _act = ref_engine.load_reference()
    scn._load_bullet_decal_assets = lambda: (np.zeros((5, 9, 7), np.uint8), np.zeros(5, np.int32),
                                             np.zeros(5, np.int32), np.zeros(5, np.int32))
    pwad, iwad = wadgen.synthetic_pair(gdscene, gdwad)
    with tempfile.TemporaryDirectory() as tmp:
        paths = []
        for name, payload in (("map.wad", pwad), ("game.wad", iwad)):
            paths.append(os.path.join(tmp, name))
            with open(paths[-1], "wb") as handle:
                handle.write(payload)
        cs = scn.compile_deathmatch_scenario(paths[0], paths[1], require_pinned_scenario=False)
    out = {"pwad_sha256": hashlib.sha256(pwad).hexdigest(), "iwad_sha256": hashlib.sha256(iwad).hexdigest(),
           "tables": summarize(cs)}
    with open(os.path.join(HERE, "golden_wad.json"), "w") as handle:
        json.dump(out, handle, indent=1)
    print("wad fixture written:", len(FIELDS), "tables")


if __name__ == "__main__":
    main()
