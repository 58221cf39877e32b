"""Seeded synthetic WAD files for the tests of the WAD / UDMF / picture readers.

No real game data exists on any machine the tests run on, so the inputs are built here, byte
by byte, from a seed: an IWAD with a palette, a colormap, PNAMES / TEXTURE1 / TEXTURE2
composites (overlapping and partly off-texture patches), pictures with holes and tall-patch
posts, flats, every sprite, weapon and status-bar lump the game tables ask for (single
rotations, all-rotation lumps and mirrored double-rotation lumps), and a PWAD whose TEXTMAP is a
grid map written as UDMF with comments, strings with escapes, floats and booleans.
"""

from __future__ import annotations

import struct

import numpy as np


def picture_bytes(rng, width, height, left, top, *, holes=True, tall=False) -> bytes:
    """A picture lump: random posts per column; with ``tall`` some posts use the relative-top rule."""

    columns = []
    for _x in range(width):
        posts = bytearray()
        y, previous = 0, -1
        while y < height:
            if holes and rng.random() < 0.3:
                y += int(rng.integers(1, 4))
                continue
            length = int(min(rng.integers(1, 9), height - y))
            top_byte = y
            if tall and previous >= 0 and y - previous <= previous and rng.random() < 0.5:
                top_byte = y - previous        # not above the previous top: read relative to it
            pixels = rng.integers(0, 256, size=length).astype(np.uint8).tobytes()
            posts += bytes((top_byte, length, 0)) + pixels + b"\0"
            previous = y
            y += length
            if holes:
                y += 1                         # posts of one column never touch, so tops strictly increase
        posts += b"\xff"
        columns.append(bytes(posts))
    header = struct.pack("<hhhh", width, height, left, top)
    table_at = 8 + 4 * width
    offsets, cursor = [], table_at
    for col in columns:
        offsets.append(cursor)
        cursor += len(col)
    return header + struct.pack(f"<{width}i", *offsets) + b"".join(columns)


def wad_bytes(identity: bytes, lumps) -> bytes:
    """``lumps``: list of (name, payload).  Directory at the end, as most tools write it."""

    body = bytearray()
    directory = bytearray()
    for name, payload in lumps:
        directory += struct.pack("<II8s", 12 + len(body), len(payload), name.encode("ascii"))
        body += payload
    return struct.pack("<4sII", identity, len(lumps), 12 + len(body)) + bytes(body) + bytes(directory)


def synthetic_iwad(tables, texture_names, flat_names, seed: int) -> bytes:
    rng = np.random.default_rng(seed)
    lumps = []
    lumps.append(("PLAYPAL", rng.integers(0, 256, size=14 * 768).astype(np.uint8).tobytes()))
    colormap = np.empty((34, 256), dtype=np.uint8)
    for row in range(34):
        colormap[row] = rng.permutation(256) if row else np.arange(256)
    lumps.append(("COLORMAP", colormap.tobytes()))
    # patches for composite textures
    patch_names = [f"PAT{i:02d}" for i in range(12)]
    pnames = struct.pack("<i", len(patch_names)) + b"".join(n.encode("ascii").ljust(8, b"\0") for n in patch_names)
    lumps.append(("PNAMES", pnames))
    patch_sizes = {}
    for i, name in enumerate(patch_names):
        w, h = int(rng.choice((16, 32, 64))), int(rng.choice((32, 64, 128)))
        patch_sizes[name] = (w, h)
        lumps.append((name, picture_bytes(rng, w, h, 0, 0, holes=(i % 3 == 0), tall=False)))

    def texture_lump(names):
        entries = []
        for name in names:
            width, height = int(rng.choice((32, 64, 128))), int(rng.choice((64, 128)))
            parts = []
            for _ in range(int(rng.integers(1, 5))):
                p = int(rng.integers(0, len(patch_names)))
                parts.append((int(rng.integers(-24, width)), int(rng.integers(-24, height)), p))
            # a full-size opaque backing patch first, so most texels are defined
            entries.append((name, width, height, [(0, 0, int(rng.integers(0, len(patch_names))))] + parts))
        blob = bytearray()
        offsets = []
        base = 4 + 4 * len(entries)
        for name, width, height, parts in entries:
            offsets.append(base + len(blob))
            blob += struct.pack("<8sIhhIh", name.encode("ascii"), 0, width, height, 0, len(parts))
            for ox, oy, p in parts:
                blob += struct.pack("<hhhhh", ox, oy, p, 1, 0)
        return struct.pack("<i", len(entries)) + struct.pack(f"<{len(entries)}i", *offsets) + bytes(blob)

    half = len(texture_names) // 2
    lumps.append(("TEXTURE1", texture_lump(texture_names[:half])))
    lumps.append(("TEXTURE2", texture_lump(texture_names[half:])))
    lumps.append(("F_START", b""))
    for name in flat_names:
        lumps.append((name, rng.integers(0, 256, size=4096).astype(np.uint8).tobytes()))
    lumps.append(("F_END", b""))
    # sprites: every request of the game tables must resolve
    lumps.append(("S_START", b""))
    have = set()

    def sprite(name, mirrored_partner=None):
        w, h = int(rng.integers(6, 20)), int(rng.integers(8, 24))
        lump = name if mirrored_partner is None else name + mirrored_partner
        lumps.append((lump, picture_bytes(rng, w, h, int(rng.integers(0, w)), int(rng.integers(0, h + 4)),
                                          tall=(len(have) % 5 == 0))))
        have.add(name)

    def rotations(prefix, frame):
        # rotations 1 and 5 on their own, 2/8, 3/7, 4/6 as mirrored pairs: the classic layout
        sprite(f"{prefix}{frame}1")
        sprite(f"{prefix}{frame}2", f"{frame}8")
        sprite(f"{prefix}{frame}3", f"{frame}7")
        sprite(f"{prefix}{frame}4", f"{frame}6")
        sprite(f"{prefix}{frame}5")

    for k, prefix in enumerate(tables.enemy_prefixes):
        for frame in sorted(set("ABCD") | set(tables.enemy_attack_frames[k]) | {tables.enemy_pain_frames[k]}):
            rotations(prefix, frame)
        for frame in sorted(set(tables.enemy_death_frames[k]) | set(tables.enemy_xdeath_frames[k])):
            if frame not in set("ABCD") | set(tables.enemy_attack_frames[k]) | {tables.enemy_pain_frames[k]}:
                sprite(f"{prefix}{frame}0")
    # a death frame that only exists as rotations (BOS2 'H' pain is rotated, 'I' death is not): covered above
    rotations("MISL", "A")
    for frame in "BCD":
        sprite(f"MISL{frame}0")
    for frame in "AB":
        sprite(f"PLSS{frame}0")
        rotations("BAL7", frame)
    for frame in "ABCDE":
        sprite(f"PLSE{frame}0")
    for frame in "CDE":
        sprite(f"BAL7{frame}0")
    for frame in "ABCDEFGHIJ":
        sprite(f"TFOG{frame}0")
    for frame in "ABCD":
        sprite(f"PUFF{frame}0")
    for name in (*tables.static_sprites, *tables.item_animation):
        if name not in have and not (name[:4] in ("MISL", "BAL7") and name[5] != "0"):
            sprite(name)
    for name in tables.weapon_patches:
        w, h = int(rng.integers(30, 90)), int(rng.integers(30, 80))
        lumps.append((name, picture_bytes(rng, w, h, -int(rng.integers(100, 200)), -int(rng.integers(60, 120)))))
    lumps.append(("S_END", b""))
    for name in tables.hud_patches:
        if name == "STBAR":
            w, h = 320, 32
        else:
            w, h = int(rng.integers(6, 30)), int(rng.integers(6, 30))
        lumps.append((name, picture_bytes(rng, w, h, 0, 0, holes=(name != "STBAR"))))
    return wad_bytes(b"IWAD", lumps)


def textmap(scene, texture_names, flat_names, seed: int) -> str:
    """UDMF text of a grid ``Scene`` (wall textures by index into ``texture_names``, flats likewise)."""

    rng = np.random.default_rng(seed)
    walls = scene.walls
    points = np.unique(walls.reshape(-1, 2), axis=0)
    index = {(float(x), float(y)): i for i, (x, y) in enumerate(points)}
    out = ["// synthetic map", 'namespace = "zdoom";', "/* vertices\n   follow */"]
    for x, y in points:
        out.append(f"vertex {{ x = {float(x):.3f}; y = {float(y):.3f}; }}")
    sides = []

    def side(wall, slot):
        sector = int(scene.wall_sectors[wall, slot])
        names = []
        for t, key in enumerate(("texturemiddle", "texturebottom", "texturetop")):
            tid = int(scene.side_textures[wall, slot, t])
            if tid >= 0:
                names.append(f'{key} = "{texture_names[tid % len(texture_names)]}";')
            elif rng.random() < 0.3:
                names.append(f'{key} = "-";')
        ox, oy = (float(v) for v in scene.side_offsets[wall, slot])
        sides.append(f"sidedef {{ sector = {sector}; {' '.join(names)} offsetx = {int(ox)}; offsety = {oy:.1f}; "
                     f'comment = "a \\"quoted\\" name"; }}')
        return len(sides) - 1

    for w in range(len(walls)):
        a = index[(float(walls[w, 0]), float(walls[w, 1]))]
        b = index[(float(walls[w, 2]), float(walls[w, 3]))]
        front = side(w, 0)
        text = f"linedef {{ v1 = {a}; v2 = {b}; sidefront = {front};"
        if scene.wall_sectors[w, 1] >= 0:
            text += f" sideback = {side(w, 1)}; twosided = true;"
            if rng.random() < 0.05:
                text += " blocking = true;"
        else:
            text += " blocking = true;"
        out.append(text + " }")
    out.extend(sides)
    for s in range(scene.num_sectors):
        floor, ceiling = (float(v) for v in scene.sector_heights[s])
        out.append(f"sector {{ heightfloor = {int(floor)}; heightceiling = {int(ceiling)}; "
                   f'texturefloor = "{flat_names[int(scene.sector_floor_tex[s]) % len(flat_names)]}"; '
                   f'textureceiling = "{flat_names[int(scene.sector_ceil_tex[s]) % len(flat_names)]}"; '
                   f"lightlevel = {int(scene.sector_lights[s])}; }}")
    for x, y, angle in scene.player_starts[:, :3]:
        out.append(f"thing {{ x = {float(x):.1f}; y = {float(y):.1f}; angle = {int(np.degrees(angle)) % 360}; type = 1; }}")
    for i, kind in enumerate((2014, 2015, 2018, 2019, 2011, 2007)):
        out.append(f"thing {{ x = {100 + 40 * i}.0; y = 1.5e2; type = {kind}; height = {8 * (i % 2)}; skill1 = true; }}")
    return "\n".join(out) + "\n"


def synthetic_pair(pkg_scene, pkg_wad, seed: int = 7):
    """``(pwad bytes, iwad bytes)``: c1's grid map as UDMF against a synthetic IWAD."""

    spec = pkg_scene.GRID_CONFIGS["c1m"]
    scene = pkg_scene.make_grid_scene(spec)
    tables = pkg_wad.GameTables()
    walls_used = int(scene.side_textures.max()) + 1
    texture_names = [f"WALL{i:02d}" for i in range(max(walls_used, 6))] + ["BFALL1", "BFALL2", "BFALL3", "BFALL4"]
    texture_names[1] = "BFALL2"      # one animated texture is referenced: its whole cycle must be compiled
    flat_names = [f"FLAT{i:02d}" for i in range(6)]
    iwad = synthetic_iwad(tables, sorted(set(texture_names)), flat_names, seed)
    text = textmap(scene, texture_names[:max(walls_used, 6)], flat_names, seed + 1)
    pwad = wad_bytes(b"PWAD", [("MAP01", b""), ("TEXTMAP", text.encode("utf-8")), ("ENDMAP", b"")])
    return pwad, iwad


def view_lanes(pkg_scene, pkg_state, scene, poses):
    """Lane records for players standing at ``poses`` (x, y, angle in radians) of any Scene."""

    lanes = np.zeros((len(poses), 32), dtype=np.int32)
    lf = lanes.view(np.float32)
    for i, (x, y, angle) in enumerate(poses):
        sector = pkg_scene.sector_at(scene, np.float32([x]), np.float32([y]))[0]
        lf[i, pkg_state.L_X], lf[i, pkg_state.L_Y], lf[i, pkg_state.L_ANGLE] = x, y, angle
        lf[i, pkg_state.L_VIEW_Z] = 41.0 + scene.sector_heights[sector, 0]
        lanes[i, pkg_state.L_X_FIXED], lanes[i, pkg_state.L_Y_FIXED] = int(x * 65536), int(y * 65536)
        bam = np.int64(round(angle / (2 * np.pi) * (1 << 32))) & 0xFFFFFFFF
        lanes[i, pkg_state.L_ANGLE_BAM] = np.uint32(bam).view(np.int32)
        lf[i, pkg_state.L_ANGLE] = np.float32(bam) * np.float32(2 * np.pi / (1 << 32))
        lanes[i, pkg_state.L_WPN_PENDING] = -1
        lanes[i, pkg_state.L_WEAPON] = i % 8
        lf[i, pkg_state.L_HEALTH] = 100.0
    return lanes
