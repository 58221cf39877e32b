"""ctypes wrapper around the CPU oracle (``gd_oracle.c``).

Test infrastructure: imported only by the tests, the smoke check and the
CPU-baseline leg of the benchmark.  ``build()`` compiles the C file with gcc;
nothing here is reachable from the product package.
"""

from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
SOURCE = os.path.join(HERE, "gd_oracle.c")
STATE_SOURCE = os.path.join(HERE, "gd_oracle_state.c")
MOVE_SOURCE = os.path.join(HERE, "gd_oracle_move.c")
LIBRARY = os.path.join(HERE, "_gd_oracle.so")

STAGE_WALLS, STAGE_SPRITES, STAGE_WEAPON, STAGE_HUD = 1, 2, 4, 8
STAGE_ALL = 15

_lib = None


def build(force: bool = False) -> str:
    headers = [os.path.join(HERE, "..", "include", h) for h in ("gradoom_b200_layout.h", "gradoom_b200.h")]
    stale = (not os.path.exists(LIBRARY)) or os.path.getmtime(LIBRARY) < max(
        os.path.getmtime(f) for f in (SOURCE, STATE_SOURCE, MOVE_SOURCE, *headers))
    if force or stale:
        subprocess.check_call(
            ["gcc", "-O2", "-ffp-contract=off", "-fno-fast-math", "-fPIC", "-shared",
             "-o", LIBRARY, SOURCE, STATE_SOURCE, MOVE_SOURCE, "-lm"])
    return LIBRARY


def lib():
    global _lib
    if _lib is None:
        build()
        _lib = ctypes.CDLL(LIBRARY)
        _lib.gd_oracle_render.restype = ctypes.c_int
        _lib.gd_oracle_resize.restype = ctypes.c_int
        _lib.gd_oracle_rgb.restype = ctypes.c_int
        _lib.gd_oracle_stack.restype = ctypes.c_int
        _lib.gd_oracle_pack_state.restype = ctypes.c_int
        _lib.gd_oracle_player_tics.restype = ctypes.c_int
    return _lib


def _ptr(a):
    return None if a is None else a.ctypes.data_as(ctypes.c_void_p)


DECAL_DTYPE = np.dtype([("serial", "<i4"), ("wall", "<i2"), ("style", "<u2"), ("along", "<f4"), ("z", "<f4")])


def render(blob, lanes, things, *, mask_hud=True, stage_mask=STAGE_ALL, depth_override=None,
           want_stages=False, decals=None):
    """Render every lane on the CPU.

    ``decals``: optional ``(N, slots)`` array of ``DECAL_DTYPE`` records (the lanes' bullet-chip rings).

    Returns a dict with ``indexed (N,240,320) u8``, ``obs (N,84,84) u8``,
    ``unowned (N,) i32`` and, on request, ``stages (N,3,208,320) u8`` (the view
    after walls + planes, after sprites, after the weapon).
    """

    blob = np.ascontiguousarray(blob, dtype=np.uint8)
    lanes = np.ascontiguousarray(lanes, dtype=np.int32)
    things = np.ascontiguousarray(things, dtype=np.int32)
    n = lanes.shape[0]
    k = things.shape[1]
    indexed = np.zeros((n, 240, 320), dtype=np.uint8)
    obs = np.zeros((n, 84, 84), dtype=np.uint8)
    unowned = np.zeros(n, dtype=np.int32)
    stages = np.zeros((n, 3, 208, 320), dtype=np.uint8) if want_stages else None
    if depth_override is not None:
        depth_override = np.ascontiguousarray(depth_override, dtype=np.float32)
    if decals is not None:
        decals = np.ascontiguousarray(decals, dtype=DECAL_DTYPE)
        assert decals.ndim == 2 and decals.shape[0] == n
        lib().gd_oracle_bind_decals(_ptr(decals), ctypes.c_int(decals.shape[1]))
    try:
        rc = lib().gd_oracle_render(_ptr(blob), _ptr(lanes), _ptr(things), ctypes.c_int(k),
                                    _ptr(depth_override), ctypes.c_int(n), ctypes.c_int(int(mask_hud)),
                                    ctypes.c_int(stage_mask), _ptr(indexed), _ptr(obs), _ptr(stages),
                                    _ptr(unowned))
    finally:
        if decals is not None:
            lib().gd_oracle_bind_decals(None, ctypes.c_int(0))
    if rc != 0:
        raise RuntimeError(f"oracle rejected the scene blob (code {rc})")
    out = {"indexed": indexed, "obs": obs, "unowned": unowned}
    if want_stages:
        out["stages"] = stages
    return out


def resize(blob, indexed):
    """Integer 320x{208,240} -> 84x84 area resize + grayscale of indexed frames."""

    blob = np.ascontiguousarray(blob, dtype=np.uint8)
    indexed = np.ascontiguousarray(indexed, dtype=np.uint8)
    n, rows = indexed.shape[0], indexed.shape[1]
    obs = np.zeros((n, 84, 84), dtype=np.uint8)
    lib().gd_oracle_resize(_ptr(blob), _ptr(indexed), ctypes.c_int(n), ctypes.c_int(rows), _ptr(obs))
    return obs


def rgb(blob, indexed, lanes=None):
    """PLAYPAL expansion; ``lanes`` carries the per-lane screen-flash state."""

    blob = np.ascontiguousarray(blob, dtype=np.uint8)
    indexed = np.ascontiguousarray(indexed, dtype=np.uint8)
    if lanes is not None:
        lanes = np.ascontiguousarray(lanes, dtype=np.int32)
    n, rows = indexed.shape[0], indexed.shape[1]
    out = np.zeros((n, rows, 320, 3), dtype=np.uint8)
    lib().gd_oracle_rgb(_ptr(blob), _ptr(lanes), _ptr(indexed), ctypes.c_int(n), ctypes.c_int(rows), _ptr(out))
    return out


def stack_update(stack, obs, reset_mask=None):
    """In-place frame-stack update: roll + append, or fill for reset lanes."""

    assert stack.dtype == np.uint8 and stack.flags.c_contiguous
    obs = np.ascontiguousarray(obs, dtype=np.uint8)
    mask = None if reset_mask is None else np.ascontiguousarray(reset_mask, dtype=np.uint8)
    lib().gd_oracle_stack(_ptr(stack), _ptr(obs), _ptr(mask), ctypes.c_int(stack.shape[0]))
    return stack


def flats(blob, lanes):
    """The complete per-pixel fallback flat layer, ``(N,208,320) u8`` (validation aid)."""

    blob = np.ascontiguousarray(blob, dtype=np.uint8)
    lanes = np.ascontiguousarray(lanes, dtype=np.int32)
    out = np.zeros((lanes.shape[0], 208, 320), dtype=np.uint8)
    lib().gd_oracle_flats(_ptr(blob), _ptr(lanes), ctypes.c_int(lanes.shape[0]), _ptr(out))
    return out


def pack_state(blob, src, max_things, *, render_screen_flashes=None):
    """Lane and thing records from an object that carries the reference engine's
    lane tensors on the CPU (the checker of the CUDA library's ``gd_pack_state``).

    Returns ``(lanes (N,32) i32, things (N,max_things,4) i32, K)``.
    """

    from gradoom_b200 import state as gdstate      # the struct layout is shared with the product binding

    es = gdstate.EngineState(src, render_screen_flashes=render_screen_flashes)
    if es.device.type != "cpu":
        raise TypeError("the oracle packs CPU tensors")
    blob = np.ascontiguousarray(blob, dtype=np.uint8)
    n = es.n
    lanes = np.zeros((n, 32), dtype=np.int32)
    things = np.zeros((n, max(max_things, 1), 4), dtype=np.int32)
    k = lib().gd_oracle_pack_state(_ptr(blob), ctypes.byref(es.struct), ctypes.c_int(max_things), _ptr(lanes),
                                   _ptr(things))
    if k < 0:
        raise RuntimeError(f"oracle rejected the state or the blob (code {k})")
    return lanes, things, int(k)


def player_tics(blob, players, buttons, tics, episode_timeout, actors=None):
    """Advance ``players (N,24) i32`` in place by ``tics`` game tics under ``buttons (N,) u32``
    (the checker of the CUDA library's ``gd_player_tics``).  ``actors``: an object with the
    reference engine's monster tensors on the CPU, or None."""

    from gradoom_b200 import state as gdstate

    blob = np.ascontiguousarray(blob, dtype=np.uint8)
    assert players.dtype == np.int32 and players.flags.c_contiguous and players.shape[1] == gdstate.PLAYER_WORDS
    buttons = np.ascontiguousarray(buttons, dtype=np.uint32)
    solid = None
    if actors is not None:
        solid = gdstate.SolidActors(actors)
        if solid.device.type != "cpu":
            raise TypeError("the oracle reads CPU tensors")
    rc = lib().gd_oracle_player_tics(_ptr(blob), _ptr(players), _ptr(buttons),
                                     None if solid is None else ctypes.byref(solid.struct),
                                     ctypes.c_int(players.shape[0]), ctypes.c_int(tics), ctypes.c_int(episode_timeout))
    if rc != 0:
        raise RuntimeError(f"oracle rejected the blob (code {rc})")
    return players
