import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import __graft_entry__ as entry  # noqa: E402

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def pkg():
    return entry.load_package()


@pytest.fixture(scope="session")
def oracle():
    return entry.load_oracle()


@pytest.fixture(scope="session")
def scenes(pkg):
    from gradoom_b200 import scene as gdscene

    cache = {}

    def get(name, ray_tables=None):
        key = (name, ray_tables is not None)
        if key not in cache:
            sc = gdscene.make_grid_scene(gdscene.GRID_CONFIGS[name])
            cache[key] = (sc, gdscene.pack_scene(sc, ray_table_override=ray_tables))
        return cache[key]

    return get


def load_golden(name):
    path = os.path.join(GOLDEN, f"golden_{name}.npz")
    if not os.path.exists(path):
        pytest.skip(f"fixture {path} not generated")
    return np.load(path)


def decal_rings(data):
    """``(N, slots, 4) int32`` gd_decal rings from the engine's ``hitscan_decal_*`` arrays of a fixture."""

    out = np.zeros((*data["decal_serial"].shape, 4), dtype=np.int32)
    out[..., 0] = data["decal_serial"]
    out[..., 1] = (data["decal_wall"].astype(np.int32) & 0xFFFF) | (data["decal_style"].astype(np.int32) << 16)
    out[..., 2] = data["decal_along"].astype(np.float32).view(np.int32)
    out[..., 3] = data["decal_z"].astype(np.float32).view(np.int32)
    return out


def pad_things(things, k):
    out = np.zeros((things.shape[0], k, 4), dtype=np.int32)
    out[:, : things.shape[1]] = things
    return out


def engine_from_fixture(data, device="cpu"):
    """An object that carries the reference engine's lane tensors, rebuilt from the
    ``state_*`` arrays of a fixture (the attribute names and dtypes are the engine's)."""

    import types

    import torch

    src = types.SimpleNamespace()
    for key in data.files:
        if key.startswith("state_"):
            setattr(src, key[len("state_"):], torch.from_numpy(np.ascontiguousarray(data[key])).to(device))
    return src


def fake_engine(n, seed=5, items=0, device="cpu", span=900.0):
    """Seeded stand-in for the reference engine's lane tensors (names, dtypes and
    shapes of src/gradoom/engine.py:1653-1934) with every actor class in use."""

    import types

    import torch

    from gradoom_b200 import state as gdstate

    g = torch.Generator().manual_seed(seed)
    counts = {"enemy_slots": 64, "projectile_slots": 32, "enemy_projectile_slots": 64, "puff_slots": 20,
              "items": items}
    e = types.SimpleNamespace()

    def rand_int(lo, hi, shape, dtype):
        return torch.randint(lo, hi, shape, generator=g).to(dtype)

    for field, attr, dtype, shape in gdstate.ENGINE_STATE_POINTERS:
        dims = (n,) if shape is None else (n, shape if isinstance(shape, int) else counts[shape])
        if dtype == torch.float32:
            t = torch.rand(dims, generator=g) * span + 20.0
        elif dtype == torch.uint8:
            t = torch.rand(dims, generator=g) < 0.15
        elif dtype == torch.int64:
            t = rand_int(0, 6, dims, torch.int64)
        else:
            t = rand_int(0, 40, dims, torch.int32) * (torch.rand(dims, generator=g) < 0.2).to(torch.int32)
        setattr(e, attr, t)
    e._x_fixed = rand_int(20 << 16, 900 << 16, (n,), torch.int64)
    e._y_fixed = rand_int(20 << 16, 900 << 16, (n,), torch.int64)
    e.x, e.y = e._x_fixed.float() / 65536, e._y_fixed.float() / 65536
    e._angle_bam = rand_int(0, 1 << 32, (n,), torch.int64)
    e.angle = e._angle_bam.float() * (2 * np.pi / (1 << 32))
    e._pitch_bam = torch.zeros(n, dtype=torch.int64)
    e._player_bob_fixed = rand_int(0, 16 << 16, (n,), torch.int64)
    e.view_z = torch.full((n,), 41.0)
    e.enemy_angle = torch.rand((n, 64), generator=g) * 6.28 - 3.14
    e.enemy_target_slot = rand_int(-2, 4, (n, 64), torch.int64)
    e.enemy_attack_phase = rand_int(0, 5, (n, 64), torch.int32)
    e.enemy_animation_tics = rand_int(0, 300, (n, 64), torch.int32)
    e.enemy_death_elapsed = rand_int(0, 80, (n, 64), torch.int32)
    e.teleport_fog_tics = rand_int(0, 73, (n, 64), torch.int32) * (torch.rand((n, 64), generator=g) < 0.05).to(torch.int32)
    e.drop_type = torch.tensor([-1, 2007, 2002, 2001])[rand_int(0, 4, (n, 64), torch.int64)]
    e.projectile_velocity_x = torch.randn((n, 32), generator=g) * 10
    e.projectile_velocity_y = torch.randn((n, 32), generator=g) * 10
    e.projectile_type = rand_int(-1, 2, (n, 32), torch.int64)
    e.projectile_impact_type = rand_int(-1, 3, (n, 32), torch.int64)
    e.enemy_projectile_velocity_x = torch.randn((n, 64), generator=g) * 10
    e.enemy_projectile_velocity_y = torch.randn((n, 64), generator=g) * 10
    e.selected_weapon = rand_int(0, 7, (n,), torch.int64)
    e.pending_weapon = rand_int(-1, 7, (n,), torch.int64)
    e.weapons = (torch.rand((n, 6), generator=g) < 0.5).float()
    e.health = rand_int(0, 201, (n,), torch.int32).float()
    e.item_animation_initial_tics = rand_int(1, 7, (n, items), torch.int32)
    e.episode_time = rand_int(1, 900, (n,), torch.int32)
    # keep the record count within the renderer's 64: a handful of slots per class
    for name, keep in (("enemy_alive", 6), ("enemy_death_tics", 5), ("teleport_fog_tics", 4), ("drop_spawned", 4),
                       ("projectile_alive", 4), ("projectile_impact_tics", 3), ("enemy_projectile_alive", 4),
                       ("enemy_projectile_impact_tics", 3), ("hitscan_puff_tics", 4)):
        t = getattr(e, name)
        t[:, keep:] = 0
    if device != "cpu":
        for attr, t in list(vars(e).items()):
            setattr(e, attr, t.to(device))
    return e
