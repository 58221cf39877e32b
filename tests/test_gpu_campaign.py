"""CUDA path against the CPU oracle on seeded random scene specifications: grid shape, room
size, texture sizes, floor range, diagonal lines, masked middle textures, split lines, bullet
chips, thing count and the status bar all vary; the players walk with the kinematics kernel
before the comparison, so some stand in doorways.  Every indexed frame and observation must be equal.  With
GD_CAMPAIGN_LOG set, one line per specification is appended to that file; GD_CAMPAIGN_SPECS and
GD_CAMPAIGN_FIRST widen or move the range of specification numbers (default: the first 24);
GD_CAMPAIGN_MAX_GRID raises the largest grid side (default 8; 16 reaches 800-wall maps, which keep fewer
tables in shared memory)."""

import dataclasses
import json
import os
from concurrent.futures import ThreadPoolExecutor

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
SPECS = int(os.environ.get("GD_CAMPAIGN_SPECS", "24"))
FIRST = int(os.environ.get("GD_CAMPAIGN_FIRST", "0"))
MAX_GRID = int(os.environ.get("GD_CAMPAIGN_MAX_GRID", "8"))
LANES = 256


def _spec(gdscene, trial):
    rng = np.random.default_rng(9000 + trial)
    return gdscene.GridSpec(
        rows=int(rng.integers(2, MAX_GRID + 1)), cols=int(rng.integers(2, MAX_GRID + 1)), room=float(rng.choice([96.0, 128.0, 192.0, 256.0, 320.0])),
        seed=300 + trial, wall_textures=int(rng.choice([4, 8, 16])), tex_w=int(rng.choice([64, 128])), tex_h=128,
        flats=int(rng.choice([2, 4, 8])), floor_max=int(rng.choice([0, 32, 64, 128])),
        diagonals=bool(rng.random() < 0.4), mid_textures=float(rng.choice([0.0, 0.0, 0.3, 0.8]))), rng


@pytest.mark.parametrize("trial", range(FIRST, FIRST + SPECS))
def test_random_scene_specification(trial, pkg, oracle):
    from gradoom_b200 import native, scene as gdscene, stepper
    from gradoom_b200.env import action_matrix

    spec, rng = _spec(gdscene, trial)
    extra = np.random.default_rng(9500 + trial)       # a generator of its own: the older draws stay as they were
    splits = 0.3 if extra.random() < 0.4 else 0.0
    chips = 24 if extra.random() < 0.5 else 0
    spec = dataclasses.replace(spec, splits=splits, decals=chips > 0)
    sc = gdscene.make_grid_scene(spec)
    blob = gdscene.pack_scene(sc)
    k = int(rng.choice([0, 4, 12, 32]))
    r = native.Renderer(blob, DEV, max(k, 1))
    producer = stepper.LaneStepper(sc, LANES, device=DEV, k_things=k, max_things=max(k, 1), seed=trial)
    producer.bind_renderer(r)
    producer.reset(torch.ones(LANES, dtype=torch.bool, device=DEV), torch.arange(LANES, device=DEV) + 5)
    table = action_matrix(DEV)
    g = torch.Generator(device=DEV).manual_seed(trial)
    steps = int(rng.integers(0, 40))
    for _ in range(steps):
        producer.step(table[torch.randint(0, 17, (LANES,), device=DEV, generator=g)])
    lanes, things = producer.render_inputs()
    host_lanes, host_things = lanes.cpu().numpy(), things.cpu().numpy()
    rings = None
    if chips:
        rings = stepper.random_decals(sc, host_lanes, chips, 64, seed=9700 + trial)
        r.bind_decals(torch.from_numpy(rings).to(DEV))
    hud = bool(trial % 2)
    obs, indexed, _ = r.frames(lanes, things, obs=True, indexed=True, mask_hud=not hud)
    r.check_status()
    chunk = 32

    def draw(i):
        part = None if rings is None else rings[i:i + chunk].view(oracle.DECAL_DTYPE)[..., 0]
        return oracle.render(blob, host_lanes[i:i + chunk], host_things[i:i + chunk], mask_hud=not hud, decals=part)

    with ThreadPoolExecutor(max_workers=min(len(os.sched_getaffinity(0)), 8)) as pool:
        parts = list(pool.map(draw, range(0, LANES, chunk)))
    want_indexed = np.concatenate([p["indexed"] for p in parts])
    want_obs = np.concatenate([p["obs"] for p in parts])
    unowned = np.concatenate([p["unowned"] for p in parts])
    wrong = ((indexed.cpu().numpy() != want_indexed).reshape(LANES, -1).any(axis=1)
             | (obs.cpu().numpy() != want_obs).reshape(LANES, -1).any(axis=1))
    log = os.environ.get("GD_CAMPAIGN_LOG")
    if log:
        with open(log, "a") as f:
            f.write(json.dumps({"trial": trial, "rows": spec.rows, "cols": spec.cols, "room": spec.room,
                                "diagonals": spec.diagonals, "mid_textures": spec.mid_textures, "things": k,
                                "split_lines": len(sc.meta.get("fragments", {})), "chips_per_lane": chips,
                                "walls": sc.num_walls, "steps_walked": steps, "status_bar": hud, "lanes": LANES,
                                "lanes_with_fallback_pixels": int((unowned > 0).sum()),
                                "mismatching_lanes": int(wrong.sum())}) + "\n")
    r.close()
    assert not wrong.any(), f"{int(wrong.sum())} of {LANES} lanes differ from the oracle"
