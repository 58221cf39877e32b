"""The WAD / UDMF / picture front end (src/gradoom/wad.py:29-164, textures.py:127-543,
scenario.py:457-1064) against tables recorded from the upstream pipeline on a seeded synthetic WAD
pair (tests/wadgen.py builds the bytes, tests/golden/make_wad_golden.py recorded the digests)."""

import hashlib
import json
import os
import struct

import numpy as np
import pytest

import wadgen
from conftest import GOLDEN


@pytest.fixture(scope="module")
def pair(pkg):
    from gradoom_b200 import scene as gdscene, wad as gdwad

    return wadgen.synthetic_pair(gdscene, gdwad)


def test_compiled_tables_equal_the_upstream_compilers(pkg, pair):
    from gradoom_b200 import wad as gdwad

    path = os.path.join(GOLDEN, "golden_wad.json")
    if not os.path.exists(path):
        pytest.skip("fixture golden_wad.json not generated")
    with open(path) as handle:
        golden = json.load(handle)
    pwad, iwad = pair
    assert hashlib.sha256(pwad).hexdigest() == golden["pwad_sha256"]       # the generator still writes the same bytes
    assert hashlib.sha256(iwad).hexdigest() == golden["iwad_sha256"]
    cs = gdwad.compile_scenario(pwad, iwad)
    different = []
    for name, want in golden["tables"].items():
        got = getattr(cs, name)
        if isinstance(want, dict):
            a = np.ascontiguousarray(got)
            have = {"dtype": str(a.dtype), "shape": list(a.shape), "sha256": hashlib.sha256(a.tobytes()).hexdigest()}
        else:
            have = got if isinstance(got, str) else list(got)
        if have != want:
            different.append(name)
    assert not different
    assert len(golden["tables"]) >= 60 and cs.raw_sprite_atlas.shape[0] > 600


def test_a_compiled_wad_renders(pkg, oracle, pair):
    """Two files in, frames out: the compiled tables become a Scene, the Scene a blob, and the CPU
    renderer draws it (the GPU parity tests cover the same blob format)."""

    from gradoom_b200 import scene as gdscene, state as gdstate, wad as gdwad

    cs = gdwad.compile_scenario(*pair)
    sc = gdscene.from_compiled_scenario(cs)
    blob = gdscene.pack_scene(sc)
    lanes = wadgen.view_lanes(gdscene, gdstate, sc, ((128.0, 128.0, 0.3), (600.0, 400.0, 2.0)))
    out = oracle.render(blob, lanes, np.zeros((2, 1, 4), dtype=np.int32), mask_hud=False)
    assert out["unowned"].max() == 0
    assert len(np.unique(out["indexed"][:, :208])) > 100 and out["indexed"][:, 208:].max() > 0


def test_archive_and_picture_errors(pkg):
    from gradoom_b200 import wad as gdwad

    with pytest.raises(ValueError):
        gdwad.WadArchive(b"short")
    with pytest.raises(ValueError):
        gdwad.WadArchive(struct.pack("<4sII", b"ZWAD", 0, 12))
    with pytest.raises(ValueError):
        gdwad.WadArchive(struct.pack("<4sII", b"PWAD", 5, 12))                  # directory past the end
    with pytest.raises(ValueError):
        gdwad.WadArchive(struct.pack("<4sII", b"PWAD", 1, 12) + struct.pack("<II8s", 0, 999, b"BIG"))
    archive = gdwad.WadArchive(wadgen.wad_bytes(b"PWAD", [("A", b"one"), ("b", b"two"), ("A", b"three")]))
    assert archive.read("a") == b"three" and archive.read("A", occurrence=0) == b"one" and "B" in archive
    with pytest.raises(KeyError):
        archive.find("MISSING")
    with pytest.raises(ValueError):
        gdwad.decode_picture(b"\0\0\0")
    with pytest.raises(ValueError):
        gdwad.decode_picture(struct.pack("<hhhh", 4, 4, 0, 0))                  # no column table
    with pytest.raises(ValueError):
        gdwad.decode_picture(struct.pack("<hhhhi", 1, 4, 0, 0, 12) + bytes((0, 2, 0, 9)))   # post runs off the lump
    rng = np.random.default_rng(1)
    tall = gdwad.decode_picture(wadgen.picture_bytes(rng, 5, 200, 2, 3, tall=True), "tall")
    assert tall.pixels.shape == (200, 5) and (tall.left, tall.top) == (2, 3) and tall.opaque[120:].any()
    assert np.array_equal(tall.mirrored().pixels, tall.pixels[:, ::-1]) and tall.mirrored().left == 5 - 2 - 1


def test_udmf_grammar(pkg):
    from gradoom_b200 import wad as gdwad

    doc = gdwad.parse_udmf('namespace = "zdoom"; // c\n/* block\ncomment */ thing { x = 1.5e2; y = -3; skill1 = true; '
                           'name = "a \\"b\\""; kind = word; }\nthing { x = .5; }')
    assert doc.namespace == "zdoom" and len(doc.blocks["thing"]) == 2
    first = doc.blocks["thing"][0]
    assert first == {"x": 150.0, "y": -3, "skill1": True, "name": 'a "b"', "kind": "word"}
    assert doc.blocks["thing"][1]["x"] == 0.5
    for bad in ('thing { x = 1 }', 'namespace = "z"; thing x', 'namespace = "z"; thing { x 1; }', "thing { x = 1; }",
                'namespace = "z"; thing { x = 1;', 'namespace = "z"; @'):
        with pytest.raises(ValueError):
            gdwad.parse_udmf(bad)


def test_sprite_rotation_lookup(pkg):
    from gradoom_b200 import wad as gdwad

    rng = np.random.default_rng(2)
    pic = wadgen.picture_bytes(rng, 4, 4, 1, 1)
    archive = gdwad.WadArchive(wadgen.wad_bytes(b"IWAD", [("TROOA1", pic), ("TROOA2A8", pic), ("TROOB0", pic),
                                                          ("TROOC1C5", pic)]))
    assert gdwad.sprite_lump(archive, "TROOA1") == ("TROOA1", False)
    assert gdwad.sprite_lump(archive, "TROOA8") == ("TROOA2A8", True)
    assert gdwad.sprite_lump(archive, "TROOA2") == ("TROOA2A8", False)
    assert gdwad.sprite_lump(archive, "TROOB5") == ("TROOB0", False)           # rotation 0 serves all
    assert gdwad.sprite_lump(archive, "TROOC5") == ("TROOC1C5", True)
    with pytest.raises(KeyError):
        gdwad.sprite_lump(archive, "TROOD1")
    with pytest.raises(ValueError):
        gdwad.sprite_lump(archive, "TROOAX")
