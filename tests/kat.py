"""Known-answer scenes restated from the upstream's WAD-free sprite tests
(tests/test_rendering.py:2649-2694 and 2844-2887): one square room, the viewer
at its centre looking along +x, tiny 3x3 sprites on the view axis."""

import dataclasses

import numpy as np

import __graft_entry__ as entry


def square_scene(sprite_values, opaque_flags):
    entry.load_package()
    from gradoom_b200 import scene as gdscene

    spec = gdscene.GridSpec(rows=1, cols=1, room=512.0, seed=9, wall_textures=2, flats=2, floor_max=0,
                            ceil_lo=128, ceil_hi=128, sprite_patches=len(sprite_values), weapon=False, hud=False)
    sc = gdscene.make_grid_scene(spec)
    p = len(sprite_values)
    atlas = np.zeros((p, 3, 3), dtype=np.uint8)
    opaque = np.zeros((p, 3, 3), dtype=np.bool_)
    for i, (value, flag) in enumerate(zip(sprite_values, opaque_flags)):
        atlas[i] = value
        opaque[i] = flag
    identity = np.broadcast_to(np.arange(256, dtype=np.uint8), (34, 256)).copy()
    return dataclasses.replace(
        sc, spr_atlas=atlas, spr_opaque=opaque, spr_widths=np.full(p, 3, dtype=np.int32),
        spr_heights=np.full(p, 3, dtype=np.int32), spr_left=np.ones(p, dtype=np.int32),
        spr_top=np.full(p, 42, dtype=np.int32), colormap=identity)


def centre_lane(things_xyz_sprite, alive=True, style=-1, bright=False):
    """Lane record for a viewer at the room centre, angle 0, eye height 41, plus thing records."""

    from gradoom_b200 import state as gdstate

    lanes = np.zeros((1, 32), dtype=np.int32)
    lf = lanes.view(np.float32)
    lf[0, gdstate.L_X] = 256.0
    lf[0, gdstate.L_Y] = 256.0
    lf[0, gdstate.L_VIEW_Z] = 41.0
    lanes[0, gdstate.L_X_FIXED] = 256 << 16
    lanes[0, gdstate.L_Y_FIXED] = 256 << 16
    lanes[0, gdstate.L_FLAGS] = 1          # player dead: no weapon, as in the upstream test
    lanes[0, gdstate.L_WPN_PENDING] = -1
    k = len(things_xyz_sprite)
    lanes[0, gdstate.L_THINGS] = k
    things = np.zeros((1, max(k, 1), 4), dtype=np.int32)
    for i, (x, y, z, sprite) in enumerate(things_xyz_sprite):
        things[0, i, :3] = np.asarray([x, y, z], dtype=np.float32).view(np.int32)
        flags = (1 if alive else 0) | (2 if bright else 0)
        word = (sprite & 0xFFFF) | (flags << 16) | ((style & 0xFF) << 24)
        things[0, i, 3] = np.asarray([word], dtype=np.uint32).view(np.int32)[0]
    return lanes, things


def transparent_case():
    sc = square_scene([10, 20], [False, True])
    things = [(256.0 + d, 256.0, 0.0, 0 if i < 4 else 1) for i, d in enumerate((64.0, 72.0, 80.0, 88.0, 96.0))]
    return sc, centre_lane(things), 20


def fog_case(tics):
    """Teleport fog at 64 units: frame = min((72 - tics) // 6, 11), sprite value 10 + frame."""

    sc = square_scene([10 + f for f in range(12)], [True] * 12)
    if tics <= 0:
        return sc, centre_lane([(320.0, 256.0, 0.0, 0)], alive=False, style=1, bright=True), None
    frame = min((72 - tics) // 6, 11)
    return sc, centre_lane([(320.0, 256.0, 0.0, frame)], style=1, bright=True), 10 + frame
