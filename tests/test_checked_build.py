"""The checked build of the library (libgradoom_b200_checked.so, -DGD_CHECKED): every index
taken from the blob or a record is range-tested before it addresses memory; an index out of
range skips its access and sets a status bit.  Corrupted inputs go to this build only -- the
regular build is never handed one."""

import numpy as np
import pytest
import torch

from conftest import decal_rings, load_golden, pad_things

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _checked(blob, k):
    from gradoom_b200 import native

    return native.Renderer(blob, DEV, k, checked=True)


def _dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).to(DEV)


def _bits(r):
    torch.cuda.synchronize()
    bits = int(r.status[0].item())
    r.status.zero_()
    return bits


@pytest.mark.parametrize("name", ["c1", "c2", "c3", "c4", "c1m", "pitch", "fallback", "c2d", "c4d", "c1k", "state", "c1s", "c4s"])
def test_fixtures_are_clean_and_equal_under_the_checked_build(name, pkg, scenes):
    data = load_golden(name)
    _sc, blob = scenes(str(data["config"]), (data["ray_offsets"], data["ray_coscorr"]))
    r = _checked(blob, 64)
    for ci in range(len(data["checkpoints"])):
        lanes, things = data[f"lanes_{ci}"], pad_things(data[f"things_{ci}"], 64)
        _, indexed, _ = r.frames(_dev(lanes), _dev(things), indexed=True)
        assert np.array_equal(indexed.cpu().numpy(), data[f"indexed_{ci}"])
    assert _bits(r) == 0


def test_bad_records_are_reported_and_contained(pkg, oracle, scenes):
    """A sprite id beyond the atlas, a thing that lies nowhere, a pose that is not a number and a
    thing count beyond the stride: each sets its bit, and every other lane equals the oracle."""

    from gradoom_b200 import native, state as gdstate, stepper

    sc, blob = scenes("c1")
    lanes, things = stepper.random_lanes(sc, 4, 4, seed=12)
    clean = oracle.render(blob, lanes, things)["indexed"]
    r = _checked(blob, 4)

    def draw(l, t):
        _, indexed, _ = r.frames(_dev(l), _dev(t), indexed=True)
        return indexed.cpu().numpy(), _bits(r)

    frames, bits = draw(lanes, things)
    assert bits == 0 and np.array_equal(frames, clean)
    # sprite id far beyond the atlas: the thing is dropped, as if it were not alive
    bad = things.copy()
    bad[2, 0, 3] = (bad[2, 0, 3] & ~0xFFFF) | 60000
    without = things.copy()
    without[2, 0, 3] &= ~(gdstate.THING_ALIVE << 16)
    frames, bits = draw(lanes, bad)
    assert bits == native.STATUS_BAD_INDEX
    assert np.array_equal(frames, oracle.render(blob, lanes, without)["indexed"])
    # a thing whose position is not a number
    bad = things.copy()
    bad[1, 1, 0] = np.float32(np.nan).view(np.int32)
    without = things.copy()
    without[1, 1, 3] &= ~(gdstate.THING_ALIVE << 16)
    frames, bits = draw(lanes, bad)
    assert bits == native.STATUS_BAD_STATE
    assert np.array_equal(frames, oracle.render(blob, lanes, without)["indexed"])
    # a pose that is not a number: that lane is drawn from the origin, the others are untouched
    bad_lanes = lanes.copy()
    bad_lanes[3, gdstate.L_X] = np.float32(np.inf).view(np.int32)
    frames, bits = draw(bad_lanes, things)
    assert bits == native.STATUS_BAD_STATE and np.array_equal(frames[:3], clean[:3])
    # more things listed than the stride holds
    bad_lanes = lanes.copy()
    bad_lanes[0, gdstate.L_THINGS] = 9
    frames, bits = draw(bad_lanes, things)
    assert bits == native.STATUS_THINGS_OVERFLOW and np.array_equal(frames[1:], clean[1:])


def _patched(pkg, blob, section, indices, value):
    from gradoom_b200 import scene as gdscene

    out = blob.copy()
    header = out[: gdscene.GD_HDR_WORDS * 4].view(np.int32)
    offset = int(header[gdscene.GD_HDR_SECTION0 + gdscene.SEC[section]])
    for index in indices:
        out[offset + 4 * index: offset + 4 * index + 4].view(np.int32)[0] = value
    return out


def test_corrupted_blobs_are_reported_not_followed(pkg, scenes):
    """A side texture past the atlas and a wall whose back sector lies beyond the scene: the
    draw completes, the bit is set, the texture / the sector is treated as absent."""

    from gradoom_b200 import native, stepper

    sc, blob = scenes("c1")
    lanes, things = stepper.random_lanes(sc, 4, 4, seed=13)
    two_sided = np.flatnonzero(sc.wall_sectors[:, 1] >= 0)
    textures = len(sc.tex_atlas)
    lower = [(int(w) * 2 + side) * 3 + 1 for w in two_sided for side in (0, 1)]
    upper = [(int(w) * 2 + side) * 3 + 2 for w in two_sided[::2] for side in (0, 1)]
    back = [int(w) * 2 + 1 for w in two_sided[::3]]
    for section, indices, value, bit in (
            ("SIDE_TEX", lower, textures + 3, native.STATUS_BAD_INDEX),
            ("SIDE_TEX", upper, textures + 40, native.STATUS_BAD_INDEX),
            ("WALL_SECTORS", back, sc.num_sectors + 5, native.STATUS_BAD_SECTOR)):
        r = _checked(_patched(pkg, blob, section, indices, value), 4)
        bits = 0
        for seed in range(6):                       # several poses, so that some lane looks at the wall
            lanes, things = stepper.random_lanes(sc, 32, 4, seed=100 + seed)
            r.frames(_dev(lanes), _dev(things), obs=True)
            bits |= _bits(r)
        assert bits & bit, section
        r.close()


def test_decal_rings_under_the_checked_build(pkg, oracle, scenes):
    """The decal fixtures are clean and equal; records with a wall index beyond the table (clamped,
    as the reference clamps it, engine.py:13799-13806), a variant beyond the atlas, a side that does
    not exist, and positions that are not numbers draw without a fault and leave the other lanes'
    frames equal to the oracle's."""

    from gradoom_b200 import stepper

    for name in ("decals_c1d", "decals_c4d", "decals_c1md", "decals_fallback"):
        data = load_golden(name)
        _sc, blob = scenes(str(data["config"]), (data["ray_offsets"], data["ray_coscorr"]))
        r = _checked(blob, 64)
        r.bind_decals(_dev(decal_rings(data)))
        _, indexed, _ = r.frames(_dev(data["lanes_0"]), _dev(pad_things(data["things_0"], 64)), indexed=True)
        assert np.array_equal(indexed.cpu().numpy(), data["indexed_0"]) and _bits(r) == 0
    sc, blob = scenes("c1d")
    lanes, things = stepper.random_lanes(sc, 4, 4, seed=14)
    rings = stepper.random_decals(sc, lanes, 50, 64, seed=15)
    clean = oracle.render(blob, lanes, things, decals=rings.view(oracle.DECAL_DTYPE)[..., 0])["indexed"]
    odd = rings.copy()
    used = np.flatnonzero(odd[0, :, 0] >= 0)
    odd[0, used[0], 1] = 30000 | (3 << 16)                      # wall 30000
    odd[0, used[1], 1] = (odd[0, used[1], 1] & 0xFFFF) | (255 << 16)   # variant 0, side 12
    r = _checked(blob, 4)
    r.bind_decals(_dev(odd))
    _, indexed, _ = r.frames(_dev(lanes), _dev(things), indexed=True)
    assert _bits(r) == 0
    assert np.array_equal(indexed.cpu().numpy(),
                          oracle.render(blob, lanes, things, decals=odd.view(oracle.DECAL_DTYPE)[..., 0])["indexed"])
    # positions that are not numbers: whatever lane 0 shows, nothing faults and lanes 1..3 are untouched
    bad = rings.copy()
    bad[0, used[2], 2] = np.float32(np.nan).view(np.int32)      # along
    bad[0, used[3], 3] = np.float32(np.inf).view(np.int32)      # height
    bad[0, used[4], 2] = np.float32(3.0e38).view(np.int32)
    r.bind_decals(_dev(bad))
    _, indexed, _ = r.frames(_dev(lanes), _dev(things), indexed=True)
    assert _bits(r) == 0
    assert np.array_equal(indexed.cpu().numpy()[1:], clean[1:])
