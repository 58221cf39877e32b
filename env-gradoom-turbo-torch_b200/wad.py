"""WAD archives, UDMF text maps and Doom picture formats: from two files to a render ``Scene``.

The host-side front end of the render path.  It reads what the reference reads
(src/gradoom/wad.py:29-164, src/gradoom/textures.py:127-543, src/gradoom/scenario.py:457-1064)
and ends in the same tables, which ``scene.from_compiled_scenario`` turns into the device blob:

* ``WadArchive``: header, lump directory, last-wins lookup by name;
* ``parse_udmf``: the TEXTMAP grammar (global assignments and blocks of assignments);
* ``decode_picture``: Doom's column/post picture format, tall-patch rule included;
* ``TextureDirectory``: PNAMES + TEXTURE1/TEXTURE2 composites, 64x64 flats as a fallback;
* ``sprite_lump``: frame/rotation lookup with mirrored double-rotation lumps;
* ``blend_tables``: ZDoom's RGB32k-based additive, translucent and shaded-decal tables;
* ``compile_scenario``: geometry, materials, sprites, weapon and status-bar tables of a UDMF
  deathmatch map, by the game tables in ``GameTables``.

Everything here is numpy on the host; nothing is on the per-step path.
"""

from __future__ import annotations

import hashlib
import re
from dataclasses import dataclass, field
from types import SimpleNamespace

import numpy as np

# ---------------------------------------------------------------------------
# WAD archive (src/gradoom/wad.py:29-84)
# ---------------------------------------------------------------------------

_DIRECTORY = np.dtype([("offset", "<u4"), ("size", "<u4"), ("name", "S8")])


@dataclass(frozen=True)
class Lump:
    name: str
    offset: int
    size: int
    ordinal: int


class WadArchive:
    """A WAD file held in memory.  ``find`` returns the last lump of a name (a later lump
    overrides an earlier one, as in the game), or the ``occurrence``-th."""

    def __init__(self, payload: bytes, *, source: str = "<memory>"):
        payload = bytes(payload)
        if len(payload) < 12:
            raise ValueError(f"{source} is too small to be a WAD")
        identity = payload[:4]
        if identity not in (b"IWAD", b"PWAD"):
            raise ValueError(f"{source} has invalid WAD identity {identity!r}")
        count, directory = (int(v) for v in np.frombuffer(payload, dtype="<u4", count=2, offset=4))
        if directory < 12 or directory + count * _DIRECTORY.itemsize > len(payload):
            raise ValueError(f"{source} has an out-of-bounds WAD directory")
        entries = np.frombuffer(payload, dtype=_DIRECTORY, count=count, offset=directory)
        beyond = np.flatnonzero(entries["offset"].astype(np.int64) + entries["size"] > len(payload))
        if beyond.size:
            raise ValueError(f"{source} lump {int(beyond[0])} extends past end of file")
        lumps = []
        for ordinal, entry in enumerate(entries):
            try:
                name = bytes(entry["name"]).split(b"\0", 1)[0].decode("ascii").upper()
            except UnicodeDecodeError as exc:
                raise ValueError(f"{source} lump {ordinal} has a non-ASCII name") from exc
            lumps.append(Lump(name, int(entry["offset"]), int(entry["size"]), ordinal))
        self._payload = payload
        self.source = source
        self.identity = identity.decode("ascii")
        self.sha256 = hashlib.sha256(payload).hexdigest()
        self.lumps = tuple(lumps)
        index: dict[str, list[Lump]] = {}
        for lump in lumps:
            index.setdefault(lump.name, []).append(lump)
        self.by_name = {name: tuple(found) for name, found in index.items()}

    @classmethod
    def from_path(cls, path) -> "WadArchive":
        with open(path, "rb") as handle:
            return cls(handle.read(), source=str(path))

    def __contains__(self, name: str) -> bool:
        return name.upper() in self.by_name

    def find(self, name: str, *, occurrence: int = -1) -> Lump:
        try:
            return self.by_name[name.upper()][occurrence]
        except (KeyError, IndexError):
            raise KeyError(f"{self.source} does not contain lump {name.upper()!r}") from None

    def read(self, lump, *, occurrence: int = -1) -> bytes:
        if not isinstance(lump, Lump):
            lump = self.find(lump, occurrence=occurrence)
        return self._payload[lump.offset: lump.offset + lump.size]


# ---------------------------------------------------------------------------
# UDMF (src/gradoom/wad.py:87-164)
# ---------------------------------------------------------------------------

@dataclass(frozen=True)
class UdmfDocument:
    namespace: str
    assignments: dict
    blocks: dict            # block name -> tuple of property dicts, in file order


_UDMF_COMMENT = re.compile(r"//[^\n]*|/\*.*?\*/", re.DOTALL)
_UDMF_LEXEME = re.compile(
    r"\s*(?:(\"(?:\\.|[^\"\\])*\")"                              # 1 string
    r"|([+-]?(?:\d+\.\d*|\.\d+|\d+)(?:[eE][+-]?\d+)?)"            # 2 number
    r"|([A-Za-z_][A-Za-z0-9_]*)"                                  # 3 identifier / keyword
    r"|([{}=;]))")                                                # 4 punctuation


def _udmf_lexemes(text: str) -> list[str]:
    text = _UDMF_COMMENT.sub("", text)
    out, at = [], 0
    while at < len(text):
        match = _UDMF_LEXEME.match(text, at)
        if match is None:
            if text[at:].strip():
                raise ValueError(f"unsupported UDMF syntax near {text[at:at + 48]!r}")
            break
        out.append(match.group(match.lastindex))
        at = match.end()
    return out


def _udmf_value(lexeme: str):
    if lexeme[0] == '"':
        return lexeme[1:-1].encode("utf-8").decode("unicode_escape")
    lowered = lexeme.casefold()
    if lowered in ("true", "false"):
        return lowered == "true"
    if any(ch in lexeme for ch in ".eE"):
        return float(lexeme)
    try:
        return int(lexeme)
    except ValueError:
        return lexeme


def parse_udmf(payload) -> UdmfDocument:
    """``name = value;`` at the top level, ``name { key = value; ... }`` blocks."""

    text = payload.decode("utf-8") if isinstance(payload, (bytes, bytearray)) else payload
    lexemes = iter(_udmf_lexemes(text))

    def need() -> str:
        try:
            return next(lexemes)
        except StopIteration:
            raise ValueError("unexpected end of UDMF document") from None

    assignments: dict = {}
    blocks: dict[str, list[dict]] = {}
    for name in lexemes:
        opener = need()
        if opener == "=":
            assignments[name] = _udmf_value(need())
            if need() != ";":
                raise ValueError(f"UDMF assignment {name!r} is missing a semicolon")
        elif opener == "{":
            properties: dict = {}
            while (key := need()) != "}":
                if need() != "=":
                    raise ValueError(f"expected '=' after UDMF property {key!r}")
                properties[key] = _udmf_value(need())
                if need() != ";":
                    raise ValueError(f"UDMF property {key!r} is missing a semicolon")
            blocks.setdefault(name, []).append(properties)
        else:
            raise ValueError(f"expected '=' or '{{' after UDMF identifier {name!r}")
    namespace = str(assignments.get("namespace", ""))
    if not namespace:
        raise ValueError("UDMF document does not declare a namespace")
    return UdmfDocument(namespace, assignments, {name: tuple(found) for name, found in blocks.items()})


# ---------------------------------------------------------------------------
# Pictures, composite textures, sprites (src/gradoom/textures.py:127-363)
# ---------------------------------------------------------------------------

@dataclass(frozen=True)
class Picture:
    name: str
    pixels: np.ndarray      # (h, w) u8 palette indices
    opaque: np.ndarray      # (h, w) bool
    left: int = 0
    top: int = 0

    @property
    def width(self) -> int:
        return int(self.pixels.shape[1])

    @property
    def height(self) -> int:
        return int(self.pixels.shape[0])

    def mirrored(self) -> "Picture":
        return Picture(f"{self.name}:FLIPPED", np.ascontiguousarray(self.pixels[:, ::-1]),
                       np.ascontiguousarray(self.opaque[:, ::-1]), self.width - self.left - 1, self.top)


def decode_picture(payload: bytes, name: str = "<patch>") -> Picture:
    """Doom's picture format: an 8-byte header, a column offset table, and per column a list of
    posts (top row, length, pad, pixels, pad) ended by 0xFF.  A post whose top row is not below
    the previous one is relative to it (the tall-patch rule)."""

    data = np.frombuffer(payload, dtype=np.uint8)
    if data.size < 8:
        raise ValueError(f"Doom patch {name!r} is truncated")
    width, height, left, top = (int(v) for v in np.frombuffer(payload, dtype="<i2", count=4))
    if width <= 0 or height <= 0 or 8 + 4 * width > data.size:
        raise ValueError(f"Doom patch {name!r} has invalid dimensions")
    starts = np.frombuffer(payload, dtype="<i4", count=width, offset=8)
    pixels = np.zeros((height, width), dtype=np.uint8)
    opaque = np.zeros((height, width), dtype=bool)
    for x in range(width):
        at = int(starts[x])
        if not 0 <= at < data.size:
            raise ValueError(f"Doom patch {name!r} column {x} is out of bounds")
        above = -1
        while True:
            if at >= data.size:
                raise ValueError(f"Doom patch {name!r} column {x} has no terminator")
            row = int(data[at])
            if row == 0xFF:
                break
            if at + 3 > data.size:
                raise ValueError(f"Doom patch {name!r} column {x} post is truncated")
            length = int(data[at + 1])
            first = at + 3
            if row <= above:
                row += above
            above = row
            if first + length + 1 > data.size:
                raise ValueError(f"Doom patch {name!r} column {x} pixels are truncated")
            lo, hi = max(row, 0), min(row + length, height)
            if lo < hi:
                pixels[lo:hi, x] = data[first + lo - row: first + hi - row]
                opaque[lo:hi, x] = True
            at = first + length + 1
    return Picture(name.upper(), pixels, opaque, left, top)


_TEXTURE_HEADER = np.dtype([("name", "S8"), ("masked", "<u4"), ("width", "<i2"), ("height", "<i2"),
                            ("columns", "<u4"), ("patches", "<i2")])
_TEXTURE_PATCH = np.dtype([("x", "<i2"), ("y", "<i2"), ("patch", "<i2"), ("stepdir", "<i2"), ("colormap", "<i2")])


class TextureDirectory:
    """PNAMES and the TEXTURE1 / TEXTURE2 composites of an IWAD."""

    def __init__(self, wad: WadArchive):
        names = wad.read("PNAMES")
        if len(names) < 4:
            raise ValueError("IWAD PNAMES lump is truncated")
        count = int(np.frombuffer(names, dtype="<i4", count=1)[0])
        if count < 0 or 4 + 8 * count > len(names):
            raise ValueError("IWAD PNAMES lump has an invalid patch count")
        self.patches = tuple(bytes(raw).split(b"\0", 1)[0].decode("ascii").upper()
                             for raw in np.frombuffer(names, dtype="S8", count=count, offset=4))
        self.textures: dict[str, tuple[int, int, tuple[tuple[int, int, int], ...]]] = {}
        for lump in ("TEXTURE1", "TEXTURE2"):
            if lump not in wad:
                continue
            raw = wad.read(lump)
            if len(raw) < 4:
                raise ValueError(f"IWAD {lump} lump is truncated")
            total = int(np.frombuffer(raw, dtype="<i4", count=1)[0])
            if total < 0 or 4 + 4 * total > len(raw):
                raise ValueError(f"IWAD {lump} has an invalid texture count")
            for index, at in enumerate(np.frombuffer(raw, dtype="<i4", count=total, offset=4)):
                at = int(at)
                if at < 0 or at + _TEXTURE_HEADER.itemsize > len(raw):
                    raise ValueError(f"IWAD {lump} texture {index} is out of bounds")
                head = np.frombuffer(raw, dtype=_TEXTURE_HEADER, count=1, offset=at)[0]
                width, height, parts = int(head["width"]), int(head["height"]), int(head["patches"])
                if width <= 0 or height <= 0 or parts < 0:
                    raise ValueError(f"IWAD {lump} texture {index} has invalid dimensions")
                first = at + _TEXTURE_HEADER.itemsize
                if first + parts * _TEXTURE_PATCH.itemsize > len(raw):
                    raise ValueError(f"IWAD {lump} texture {index} patches are truncated")
                placed = np.frombuffer(raw, dtype=_TEXTURE_PATCH, count=parts, offset=first)
                if parts and not ((placed["patch"] >= 0) & (placed["patch"] < len(self.patches))).all():
                    raise ValueError(f"IWAD {lump} texture {index} references invalid PNAMES index")
                name = bytes(head["name"]).split(b"\0", 1)[0].decode("ascii").upper()
                self.textures[name] = (width, height, tuple((int(p["x"]), int(p["y"]), int(p["patch"])) for p in placed))

    def decode(self, wad: WadArchive, name: str) -> Picture:
        """A composite wall texture (patches pasted in order, later over earlier, transparent
        texels skipped), or a raw 64x64 flat of that name."""

        name = name.upper()
        if name not in self.textures:
            try:
                raw = wad.read(name)
            except KeyError:
                raw = b""
            if len(raw) != 64 * 64:
                raise KeyError(f"IWAD has no wall texture or 64x64 flat {name!r}")
            flat = np.frombuffer(raw, dtype=np.uint8).reshape(64, 64).copy()
            return Picture(name, flat, np.ones((64, 64), dtype=bool))
        width, height, placed = self.textures[name]
        pixels = np.zeros((height, width), dtype=np.uint8)
        opaque = np.zeros((height, width), dtype=bool)
        for ox, oy, patch_index in placed:
            patch = decode_picture(wad.read(self.patches[patch_index]), self.patches[patch_index])
            x0, y0 = max(ox, 0), max(oy, 0)
            x1, y1 = min(ox + patch.width, width), min(oy + patch.height, height)
            if x0 >= x1 or y0 >= y1:
                continue
            src = (slice(y0 - oy, y1 - oy), slice(x0 - ox, x1 - ox))
            solid = patch.opaque[src]
            pixels[y0:y1, x0:x1][solid] = patch.pixels[src][solid]
            opaque[y0:y1, x0:x1][solid] = True
        return Picture(name, pixels, opaque)


def _stack(pictures, *, with_offsets: bool):
    h = max((p.height for p in pictures), default=1)
    w = max((p.width for p in pictures), default=1)
    atlas = np.zeros((len(pictures), h, w), dtype=np.uint8)
    opaque = np.zeros((len(pictures), h, w), dtype=bool)
    for i, p in enumerate(pictures):
        atlas[i, :p.height, :p.width] = p.pixels
        opaque[i, :p.height, :p.width] = p.opaque
    sizes = (np.asarray([p.width for p in pictures], dtype=np.int32), np.asarray([p.height for p in pictures], dtype=np.int32))
    if not with_offsets:
        return atlas, opaque, *sizes
    return (atlas, opaque, *sizes, np.asarray([p.left for p in pictures], dtype=np.int32),
            np.asarray([p.top for p in pictures], dtype=np.int32))


def indexed_atlas(wad: WadArchive, names) -> tuple[np.ndarray, np.ndarray, np.ndarray]:
    """``(atlas (T,H,W) u8, widths, heights)`` of wall textures and flats, palette indices kept."""

    directory = TextureDirectory(wad)
    atlas, _opaque, widths, heights = _stack([directory.decode(wad, name) for name in names], with_offsets=False)
    return atlas, widths, heights


def sprite_lump(wad: WadArchive, request: str) -> tuple[str, bool]:
    """The lump that holds sprite ``PREFIX + frame + rotation`` and whether it is used mirrored.
    A lump name carries one frame/rotation pair, or two (the second mirrored); rotation 0 serves
    every rotation when no exact one exists.  First match in directory order."""

    request = request.upper()
    if len(request) != 6 or not request[5].isdigit():
        raise ValueError(f"sprite request must be PREFIX+frame+rotation, got {request!r}")
    prefix, frame, rotation = request[:4], request[4], request[5]
    any_rotation = None
    for lump in wad.lumps:
        name = lump.name
        if len(name) < 6 or name[:4] != prefix:
            continue
        pairs = [(name[4], name[5], False)]
        if len(name) >= 8:
            pairs.append((name[6], name[7], True))
        for f, r, mirrored in pairs:
            if f != frame:
                continue
            if r == rotation:
                return name, mirrored
            if r == "0":
                any_rotation = (name, mirrored)
    if any_rotation is None:
        raise KeyError(f"IWAD has no sprite frame {request!r}")
    return any_rotation


def indexed_sprite_atlas(wad: WadArchive, requests):
    """``(names, atlas, opaque, widths, heights, left, top)`` of sprite frames in request order."""

    pictures = []
    for request in requests:
        lump, mirrored = sprite_lump(wad, request)
        picture = decode_picture(wad.read(lump), lump)
        pictures.append(picture.mirrored() if mirrored else picture)
    return (tuple(p.name for p in pictures), *_stack(pictures, with_offsets=True))


def indexed_patch_atlas(wad: WadArchive, names):
    """The same for pictures addressed by their lump name (weapon frames, status-bar patches)."""

    names = tuple(name.upper() for name in names)
    return (names, *_stack([decode_picture(wad.read(name), name) for name in names], with_offsets=True))


# ---------------------------------------------------------------------------
# Blend tables (src/gradoom/scenario.py:214-277; ZDoom's RGB32k / Col2RGB8 scheme)
# ---------------------------------------------------------------------------

def blend_tables(playpal: np.ndarray):
    """``(additive (2,256,256), translucent (256,256), decal_opacity (32,256), black_shade (65,256))``.

    Colours are mixed in a 5-bit-per-channel space: a palette colour scaled by a level 0..64 is
    packed as three 10-bit fields (``g | r << 20 | b << 10`` after ``>> 4``), sums are clamped per
    field, and the result picks the nearest palette entry (indices 1..254) from a 32x32x32 table.
    """

    palette = np.asarray(playpal, dtype=np.int64).reshape(256, 3)
    grid = np.arange(32, dtype=np.int64)
    level = (grid << 3) | (grid >> 2)
    r, g, b = np.meshgrid(level, level, level, indexing="ij")
    targets = np.stack((r, g, b), axis=-1).reshape(-1, 3)
    distance = ((targets[:, None, :] - palette[None, 1:255, :]) ** 2).sum(axis=2)
    nearest = (np.argmin(distance, axis=1) + 1).astype(np.uint8)          # index r * 1024 + g * 32 + b

    def packed(scale: int) -> np.ndarray:
        word = (((palette[:, 0] * scale) >> 4) << 20) | ((palette[:, 1] * scale) >> 4) | (((palette[:, 2] * scale) >> 4) << 10)
        return word if scale in (0, 64) else word & 0x3FEFFBFF

    def lookup(word: np.ndarray) -> np.ndarray:
        return nearest[(word & (word >> 15)).astype(np.int64)]

    additive = np.empty((2, 256, 256), dtype=np.uint8)
    behind = packed(64)[:, None]
    for style, scale in enumerate((48, 64)):
        total = packed(scale)[None, :] + behind
        carry = total & 0x40100400
        clamped = ((total | 0x01F07C1F) & 0x3FFFFFFF) | (carry - (carry >> 5))
        additive[style] = lookup(clamped)
    translucent = lookup((packed(32)[None, :] + packed(32)[:, None]) | 0x01F07C1F)
    texel = np.arange(256, dtype=np.int64)
    shade = np.arange(32, dtype=np.int64)[:, None]
    decal_opacity = np.minimum(((texel + 2) * ((32 - shade) * 256 // 32 * 13) + 256) >> 14, 64).astype(np.uint8)
    black = np.stack([lookup(packed(64 - opacity) | 0x01F07C1F) for opacity in range(65)])
    return additive, translucent, decal_opacity, black


# ---------------------------------------------------------------------------
# Game tables: which lumps make up the actors, the weapon and the status bar
# (src/gradoom/scenario.py:62-212, 727-888; the frame letters and durations are Doom's own
# actor and weapon state definitions)
# ---------------------------------------------------------------------------

def _cycle(*steps):
    return tuple(steps)


@dataclass(frozen=True)
class GameTables:
    enemy_prefixes: tuple = ("POSS", "SPOS", "PLAY", "CPOS", "SARG", "BOS2")
    enemy_attack_frames: tuple = ("EFEF", "EFEF", "EFEF", "EFEF", "EFGH", "EFGH")
    enemy_pain_frames: str = "GGGGHH"
    enemy_death_frames: tuple = ("HIJKL", "HIJKL", "HIJKLMN", "HIJKLMN", "IJKLMN", "IJKLMNO")
    enemy_death_durations: tuple = ((5, 5, 5, 5, 1), (5, 5, 5, 5, 1), (10, 10, 10, 10, 10, 10, 1),
                                    (5, 5, 5, 5, 5, 5, 1), (8, 8, 4, 4, 4, 1), (8, 8, 8, 8, 8, 8, 1))
    enemy_xdeath_frames: tuple = ("MNOPQRSTU", "MNOPQRSTU", "OPQRSTUVW", "OPQRST", "IJKLMN", "IJKLMNO")
    enemy_xdeath_durations: tuple = ((5,) * 8 + (1,), (5,) * 8 + (1,), (5,) * 8 + (1,), (5,) * 5 + (1,),
                                     (8, 8, 4, 4, 4, 1), (8, 8, 8, 8, 8, 8, 1))
    projectile_explosions: tuple = (("MISLB0", "MISLC0", "MISLD0"), tuple(f"PLSE{f}0" for f in "ABCDE"),
                                    tuple(f"BAL7{f}0" for f in "CDE"))
    projectile_explosion_durations: tuple = ((8, 6, 4), (4, 4, 4, 4, 4), (6, 6, 6))
    teleport_fog: tuple = tuple(f"TFOG{f}0" for f in "ABABCDEFGHIJ")
    bullet_puffs: tuple = tuple(f"PUFF{f}0" for f in "ABCD")
    static_sprites: tuple = ("STIMA0", "MEDIA0", "BON1A0", "BON2A0", "ARM1A0", "ARM2A0", "CLIPA0", "AMMOA0", "SBOXA0",
                             "BROKA0", "CELPA0", "CSAWA0", "SHOTA0", "SGN2A0", "MGUNA0", "LAUNA0", "PLASA0", "MISLA1",
                             "PLSSA0", "BAL7A1")
    item_animation: tuple = ("BON1B0", "BON1C0", "BON1D0", "BON2B0", "BON2C0", "BON2D0", "ARM1B0", "ARM2B0")
    weapon_patches: tuple = (
        "PUNGA0", "PUNGB0", "PUNGC0", "PUNGD0", "SAWGA0", "SAWGB0", "SAWGC0", "SAWGD0", "PISGA0", "PISGB0", "PISGC0",
        "PISFA0", "SHTGA0", "SHTGB0", "SHTGC0", "SHTGD0", "SHTFA0", "SHTFB0", *(f"SHT2{f}0" for f in "ABCDEFGHIJ"),
        "CHGGA0", "CHGGB0", "CHGFA0", "CHGFB0", "MISGA0", "MISGB0", *(f"MISF{f}0" for f in "ABCD"), "PLSGA0", "PLSGB0",
        "PLSFA0", "PLSFB0")
    weapon_ready: tuple = ("PUNGA0", "SAWGC0", "PISGA0", "SHTGA0", "SHT2A0", "CHGGA0", "MISGA0", "PLSGA0")
    weapon_idle_override: dict = field(default_factory=lambda: {(1, 0): "SAWGC0", (1, 1): "SAWGD0"})
    weapon_cooldown_tics: int = 61
    # weapon -> firing sequence (frame, tics), first frame first
    weapon_cycles: dict = field(default_factory=lambda: {
        0: _cycle(("PUNGB0", 4), ("PUNGC0", 4), ("PUNGD0", 5), ("PUNGC0", 4), ("PUNGB0", 4)),
        1: _cycle(("SAWGA0", 4), ("SAWGB0", 3)),
        2: _cycle(("PISGA0", 4), ("PISGB0", 6), ("PISGC0", 4), ("PISGB0", 4)),
        3: _cycle(("SHTGA0", 3), ("SHTGA0", 7), ("SHTGB0", 5), ("SHTGC0", 5), ("SHTGD0", 4), ("SHTGC0", 5),
                  ("SHTGB0", 5), ("SHTGA0", 3), ("SHTGA0", 6)),
        4: _cycle(("SHT2A0", 3), ("SHT2A0", 7), ("SHT2B0", 7), ("SHT2C0", 7), ("SHT2D0", 7), ("SHT2E0", 7),
                  ("SHT2F0", 7), ("SHT2G0", 6), ("SHT2H0", 6), ("SHT2A0", 4)),
        5: _cycle(("CHGGA0", 4), ("CHGGB0", 3)),
        6: _cycle(("MISGB0", 19)),
        7: _cycle(("PLSGA0", 3), ("PLSGB0", 19)),
    })
    # (weapon, parity or None for both) -> muzzle flash sequence (frame or None, tics, extra light)
    weapon_flashes: dict = field(default_factory=lambda: {
        (2, None): _cycle((None, 4, 0), ("PISFA0", 7, 1), (None, 7, 0)),
        (3, None): _cycle((None, 3, 0), ("SHTFA0", 4, 1), ("SHTFB0", 3, 2), (None, 33, 0)),
        (4, None): _cycle((None, 3, 0), ("SHT2I0", 4, 1), ("SHT2J0", 3, 2), (None, 51, 0)),
        (6, None): _cycle(("MISFA0", 3, 1), ("MISFB0", 4, 1), ("MISFC0", 4, 2), ("MISFD0", 4, 2), (None, 4, 0)),
        (7, 0): _cycle(("PLSFB0", 4, 1), (None, 18, 0)),
        (7, 1): _cycle(("PLSFA0", 4, 1), (None, 18, 0)),
        (5, 1): _cycle(("CHGFA0", 7, 1)),
        (5, 0): _cycle(("CHGFB0", 7, 2)),
    })
    hud_patches: tuple = (
        "STBAR", "STARMS", *(f"STTNUM{d}" for d in range(10)), "STTPRCNT",
        *(f"STFST{pain}{look}" for pain in range(5) for look in range(3)), *(f"STYSNUM{d}" for d in range(10)),
        *(f"STGNUM{d}" for d in range(2, 8)), *(f"STFTR{pain}0" for pain in range(5)),
        *(f"STFKILL{pain}" for pain in range(5)), *(f"STFTL{pain}0" for pain in range(5)),
        *(f"STFOUCH{pain}" for pain in range(5)), *(f"STFEVL{pain}" for pain in range(5)), "STFDEAD0")
    texture_animations: tuple = (("BFALL1", "BFALL2", "BFALL3", "BFALL4"), ("BLOOD1", "BLOOD2", "BLOOD3"))


def _padded_frames(frames_per_kind, durations_per_kind):
    most = max(len(frames) for frames in frames_per_kind)
    counts = np.asarray([len(frames) for frames in frames_per_kind], dtype=np.int32)
    durations = np.zeros((len(frames_per_kind), most), dtype=np.int32)
    for kind, row in enumerate(durations_per_kind):
        durations[kind, :len(row)] = row
    names = [[frames[min(i, len(frames) - 1)] for i in range(most)] for frames in frames_per_kind]
    return names, counts, durations


def weapon_frame_tables(tables: GameTables):
    """``(frame_ids, flash_ids, flash_lights)``, each ``(8, 2, cooldown + 1) int32``: the weapon
    picture, the muzzle-flash picture (-1 none) and the extra light for every (weapon, fire
    parity, tics left in the firing sequence); slot 0 is the idle frame."""

    patch = {name: i for i, name in enumerate(tables.weapon_patches)}
    tics = tables.weapon_cooldown_tics + 1
    frames = np.empty((8, 2, tics), dtype=np.int32)
    flashes = np.full((8, 2, tics), -1, dtype=np.int32)
    lights = np.zeros((8, 2, tics), dtype=np.int32)
    for weapon, ready in enumerate(tables.weapon_ready):
        frames[weapon] = patch[ready]

    def lay(sequence, write):
        left = sum(step[1] for step in sequence)
        for step in sequence:
            span = step[1]
            write(step, slice(left - span + 1, left + 1))
            left -= span

    for weapon, sequence in tables.weapon_cycles.items():
        for parity in (0, 1):
            lay(sequence, lambda step, where: frames.__setitem__((weapon, parity, where), patch[step[0]]))
    for (weapon, parity), sequence in tables.weapon_flashes.items():
        for p in ((0, 1) if parity is None else (parity,)):
            def write(step, where, weapon=weapon, p=p):
                if step[0] is not None:
                    flashes[weapon, p, where] = patch[step[0]]
                lights[weapon, p, where] = step[2]
            lay(sequence, write)
    for (weapon, parity), name in tables.weapon_idle_override.items():
        frames[weapon, parity, 0] = patch[name]
    return frames, flashes, lights


# ---------------------------------------------------------------------------
# Scenario compiler (src/gradoom/scenario.py:457-1064)
# ---------------------------------------------------------------------------

def _blocks(document: UdmfDocument, name: str):
    if name not in document.blocks:
        raise ValueError(f"deathmatch TEXTMAP has no {name!r} blocks")
    return document.blocks[name]


def _texture_name(value) -> str:
    value = str(value).upper()
    return "" if value in ("", "-") else value


def compile_scenario(scenario_wad, iwad, *, tables: GameTables | None = None, decal_chips: dict | None = None):
    """Compile a UDMF deathmatch map (a PWAD with a TEXTMAP lump) against an IWAD into the table
    set of the reference's ``CompiledScenario`` (same field names, same values); feed the result
    to ``scene.from_compiled_scenario``.  ``scenario_wad`` / ``iwad``: paths, bytes or
    ``WadArchive``.  ``decal_chips``: the bullet-chip bitmaps (``atlas``, ``heights``, ``left``,
    ``top``), which live outside both WADs; without them the decal layer stays empty."""

    tables = tables or GameTables()
    scenario = _archive(scenario_wad)
    game = _archive(iwad)
    if scenario.identity != "PWAD":
        raise ValueError("deathmatch scenario must be a PWAD")
    if game.identity != "IWAD":
        raise ValueError("base game data must be an IWAD")
    document = parse_udmf(scenario.read("TEXTMAP"))
    vertices_raw, lines, sides = _blocks(document, "vertex"), _blocks(document, "linedef"), _blocks(document, "sidedef")
    sectors, things = _blocks(document, "sector"), _blocks(document, "thing")

    vertices = np.asarray([(float(v["x"]), float(v["y"])) for v in vertices_raw], dtype=np.float32)
    side_sector = np.asarray([int(s.get("sector", -1)) for s in sides], dtype=np.int32)
    L = len(lines)
    walls = np.empty((L, 4), dtype=np.float32)
    wall_sectors = np.full((L, 2), -1, dtype=np.int32)
    side_names = [[["", "", ""], ["", "", ""]] for _ in range(L)]
    side_offsets = np.zeros((L, 2, 2), dtype=np.float32)
    first_name = [""] * L
    first_offset = np.zeros((L, 2), dtype=np.float32)
    blocking = []
    for i, line in enumerate(lines):
        a, b = int(line["v1"]), int(line["v2"])
        if not (0 <= a < len(vertices) and 0 <= b < len(vertices)):
            raise ValueError(f"linedef {i} references an invalid vertex")
        walls[i] = (*vertices[a], *vertices[b])
        pair = (int(line.get("sidefront", -1)), int(line.get("sideback", -1)))
        if max(pair) >= len(sides):
            raise ValueError(f"linedef {i} references an invalid sidedef")
        for slot, s in enumerate(pair):
            if s < 0:
                continue
            wall_sectors[i, slot] = side_sector[s]
            side = sides[s]
            side_offsets[i, slot] = (float(side.get("offsetx", 0)), float(side.get("offsety", 0)))
            names = [_texture_name(side.get(key, "")) for key in ("texturemiddle", "texturebottom", "texturetop")]
            side_names[i][slot] = names
            visible = next((n for n in names if n), "")
            if visible and not first_name[i]:
                first_name[i] = visible
                first_offset[i] = side_offsets[i, slot]
        if pair[1] < 0 or bool(line.get("blocking", False)):
            if pair[0] < 0:
                raise ValueError(f"blocking linedef {i} has no front sidedef")
            if not first_name[i]:
                raise ValueError(f"blocking linedef {i} has no visible wall texture")
            blocking.append(i)

    floor_names = tuple(str(s.get("texturefloor", "")).upper() for s in sectors)
    ceiling_names = tuple(str(s.get("textureceiling", "")).upper() for s in sectors)
    if not all(floor_names) or not all(ceiling_names):
        raise ValueError("every deathmatch sector must declare floor and ceiling textures")
    used = {n for n in first_name if n} | {n for line in side_names for side in line for n in side if n}
    used |= set(floor_names) | set(ceiling_names)
    for animation in tables.texture_animations:
        if used & set(animation):
            used |= set(animation)
    texture_names = tuple(sorted(used))
    texture_id = {name: i for i, name in enumerate(texture_names)}
    texture_index_atlas, texture_widths, texture_heights = indexed_atlas(game, texture_names)

    # sprites, in the reference's request order
    requests: list[str] = []

    def want(name: str) -> int:
        requests.append(name)
        return len(requests) - 1

    kinds = range(len(tables.enemy_prefixes))
    walk = np.empty((len(tables.enemy_prefixes), 4, 8), dtype=np.int32)
    attack = np.empty_like(walk)
    for k in kinds:
        prefix = tables.enemy_prefixes[k]
        for fi, f in enumerate("ABCD"):
            for r in range(1, 9):
                walk[k, fi, r - 1] = want(f"{prefix}{f}{r}")
        for fi, f in enumerate(tables.enemy_attack_frames[k]):
            for r in range(1, 9):
                attack[k, fi, r - 1] = want(f"{prefix}{f}{r}")
    death_names, death_counts, death_durations = _padded_frames(tables.enemy_death_frames, tables.enemy_death_durations)
    death = np.asarray([[want(f"{tables.enemy_prefixes[k]}{f}0") for f in death_names[k]] for k in kinds], dtype=np.int32)
    xdeath_names, xdeath_counts, xdeath_durations = _padded_frames(tables.enemy_xdeath_frames, tables.enemy_xdeath_durations)
    xdeath = np.asarray([[want(f"{tables.enemy_prefixes[k]}{f}0") for f in xdeath_names[k]] for k in kinds], dtype=np.int32)
    pain = np.asarray([[want(f"{tables.enemy_prefixes[k]}{tables.enemy_pain_frames[k]}{r}") for r in range(1, 9)]
                       for k in kinds], dtype=np.int32)
    flight = np.empty((3, 2, 8), dtype=np.int32)
    for r in range(1, 9):
        flight[0, :, r - 1] = want(f"MISLA{r}")
        flight[1, 0, r - 1] = want("PLSSA0")
        flight[1, 1, r - 1] = want("PLSSB0")
        flight[2, 0, r - 1] = want(f"BAL7A{r}")
        flight[2, 1, r - 1] = want(f"BAL7B{r}")
    expl_names, expl_counts, expl_durations = _padded_frames(tables.projectile_explosions,
                                                             tables.projectile_explosion_durations)
    explosion = np.asarray([[want(name) for name in row] for row in expl_names], dtype=np.int32)
    fog = np.asarray([want(name) for name in tables.teleport_fog], dtype=np.int32)
    puff = np.asarray([want(name) for name in tables.bullet_puffs], dtype=np.int32)
    static = np.asarray([want(name) for name in tables.static_sprites], dtype=np.int32)
    item_animation = np.asarray([want(name) for name in tables.item_animation], dtype=np.int32)
    sprite_names, spr_atlas, spr_opaque, spr_w, spr_h, spr_left, spr_top = indexed_sprite_atlas(game, requests)

    _names, wpn_atlas, wpn_opaque, wpn_w, wpn_h, wpn_left, wpn_top = indexed_patch_atlas(game, tables.weapon_patches)
    wpn_frames, wpn_flashes, wpn_lights = weapon_frame_tables(tables)
    hud_names, hud_atlas, hud_opaque, hud_w, hud_h, hud_left, hud_top = indexed_patch_atlas(game, tables.hud_patches)

    side_ids = np.full((L, 2, 3), -1, dtype=np.int32)
    for i, line in enumerate(side_names):
        for slot, names in enumerate(line):
            for t, name in enumerate(names):
                if name:
                    side_ids[i, slot, t] = texture_id[name]
    edge_mask = np.zeros((len(sectors), L), dtype=bool)
    for i, (front, back) in enumerate(wall_sectors):
        if front >= 0 and front == back:
            continue                                   # a line inside one sector bounds nothing
        if front >= 0:
            edge_mask[front, i] = True
        if back >= 0:
            edge_mask[back, i] = True
    starts = np.asarray([(float(t["x"]), float(t["y"]), float(t.get("angle", 0))) for t in things
                         if int(t.get("type", -1)) == 1], dtype=np.float32)
    if not len(starts):
        raise ValueError("deathmatch scenario contains no player starts")
    items = [t for t in things if int(t.get("type", -1)) != 1]
    playpal = game.read("PLAYPAL")
    if len(playpal) < 768:
        raise ValueError("IWAD PLAYPAL lump is too small")
    playpal = np.frombuffer(playpal[:768], dtype=np.uint8).reshape(256, 3).copy()
    colormap = game.read("COLORMAP")
    if len(colormap) < 34 * 256:
        raise ValueError("IWAD COLORMAP lump is too small")
    colormap = np.frombuffer(colormap[:34 * 256], dtype=np.uint8).reshape(34, 256).copy()
    additive, translucent, decal_opacity, decal_black = blend_tables(playpal)
    chips = decal_chips or {}
    return SimpleNamespace(
        scenario_sha256=scenario.sha256, iwad_sha256=game.sha256, namespace=document.namespace,
        vertices=vertices, wall_segments=walls, blocking_wall_indices=np.asarray(blocking, dtype=np.int32),
        blocking_segments=walls[blocking].reshape(-1, 4).copy(),
        wall_texture_ids=np.asarray([texture_id[n] if n else -1 for n in first_name], dtype=np.int32),
        wall_texture_offsets=first_offset, wall_side_texture_ids=side_ids, wall_side_texture_offsets=side_offsets,
        wall_sectors=wall_sectors, sector_edge_mask=edge_mask,
        sector_heights=np.asarray([(float(s.get("heightfloor", 0)), float(s.get("heightceiling", 128))) for s in sectors],
                                  dtype=np.float32),
        sector_lights=np.asarray([int(s.get("lightlevel", 160)) for s in sectors], dtype=np.int16),
        sector_floor_texture_ids=np.asarray([texture_id[n] for n in floor_names], dtype=np.int32),
        sector_ceiling_texture_ids=np.asarray([texture_id[n] for n in ceiling_names], dtype=np.int32),
        player_starts=starts,
        item_spawns=np.asarray([(float(t["x"]), float(t["y"]), float(t.get("height", 0))) for t in items],
                               dtype=np.float32).reshape(-1, 3),
        item_types=np.asarray([int(t["type"]) for t in items], dtype=np.int32),
        playpal=playpal, colormap=colormap, texture_names=texture_names, texture_index_atlas=texture_index_atlas,
        texture_widths=texture_widths, texture_heights=texture_heights,
        raw_sprite_names=sprite_names, raw_sprite_atlas=spr_atlas, raw_sprite_opaque=spr_opaque,
        raw_sprite_widths=spr_w, raw_sprite_heights=spr_h, raw_sprite_left_offsets=spr_left, raw_sprite_top_offsets=spr_top,
        enemy_walk_sprite_ids=walk, enemy_attack_sprite_ids=attack, enemy_pain_sprite_ids=pain,
        enemy_death_sprite_ids=death, enemy_death_frame_counts=death_counts, enemy_death_frame_durations=death_durations,
        enemy_xdeath_sprite_ids=xdeath, enemy_xdeath_frame_counts=xdeath_counts,
        enemy_xdeath_frame_durations=xdeath_durations,
        raw_projectile_flight_sprite_ids=flight, raw_projectile_explosion_sprite_ids=explosion,
        projectile_explosion_frame_counts=expl_counts, projectile_explosion_frame_durations=expl_durations,
        raw_teleport_fog_sprite_ids=fog, raw_bullet_puff_sprite_ids=puff, raw_static_sprite_ids=static,
        raw_item_animation_sprite_ids=item_animation,
        projectile_additive_luts=additive, sprite_translucent_lut=translucent,
        bullet_decal_opacity_lut=decal_opacity, bullet_decal_black_lut=decal_black,
        bullet_decal_atlas=chips.get("atlas"), bullet_decal_heights=chips.get("heights"),
        bullet_decal_left_offsets=chips.get("left"), bullet_decal_top_offsets=chips.get("top"),
        native_weapon_patch_atlas=wpn_atlas, native_weapon_patch_opaque=wpn_opaque, native_weapon_patch_widths=wpn_w,
        native_weapon_patch_heights=wpn_h, native_weapon_patch_left_offsets=wpn_left,
        native_weapon_patch_top_offsets=wpn_top, native_weapon_frame_ids=wpn_frames,
        native_weapon_flash_ids=wpn_flashes, native_weapon_flash_lights=wpn_lights,
        hud_patch_names=hud_names, hud_patch_atlas=hud_atlas, hud_patch_opaque=hud_opaque, hud_patch_widths=hud_w,
        hud_patch_heights=hud_h, hud_patch_left_offsets=hud_left, hud_patch_top_offsets=hud_top,
    )


def _archive(source) -> WadArchive:
    if isinstance(source, WadArchive):
        return source
    if isinstance(source, (bytes, bytearray, memoryview)):
        return WadArchive(bytes(source))
    return WadArchive.from_path(source)
