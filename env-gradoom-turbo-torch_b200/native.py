"""ctypes binding of the CUDA library's C ABI (include/gradoom_b200.h).

There is no CPU fallback: if the shared library is missing or a call fails the
caller gets an exception.  PyTorch only provides device memory and streams.
"""

from __future__ import annotations

import ctypes
import os

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
LIBRARY = os.path.join(HERE, "csrc", "libgradoom_b200.so")
# the same sources compiled with -DGD_CHECKED: range tests on every index, for debugging state producers
CHECKED_LIBRARY = os.path.join(HERE, "csrc", "libgradoom_b200_checked.so")

GD_OK = 0
STATUS_EVENT_OVERFLOW = 1
STATUS_THINGS_OVERFLOW = 2
STATUS_BAD_SECTOR = 4
STATUS_BAD_INDEX = 8
STATUS_BAD_STATE = 16

EXPORTS = (
    "gd_error_string", "gd_renderer_create", "gd_renderer_destroy", "gd_renderer_scratch_bytes",
    "gd_renderer_ctas", "gd_renderer_shared_bytes", "gd_renderer_shared_bytes_view", "gd_render_step", "gd_render_reset", "gd_render_frames",
    "gd_render_step_frames", "gd_render_step_host", "gd_render_step_ring", "gd_render_reset_ring", "gd_static_scratch_bytes", "gd_static_max_walls", "gd_render_step_static",
    "gd_pack_state_scratch_bytes", "gd_pack_state", "gd_player_tics", "gd_renderer_bind_decals", "gd_probe_libm",
)

_libs = {}


class NativeError(RuntimeError):
    pass


def load(checked: bool = False) -> ctypes.CDLL:
    """Load libgradoom_b200.so (or its checked build); raise if it has not been built."""

    path = CHECKED_LIBRARY if checked else LIBRARY
    if path not in _libs:
        if not os.path.exists(path):
            raise NativeError(
                f"{path} is missing: build it with __graft_entry__.build() "
                "(nvcc, sm_100a). This package has no CPU or PyTorch fallback.")
        lib = ctypes.CDLL(path)
        vp, ci, sz = ctypes.c_void_p, ctypes.c_int, ctypes.c_size_t
        lib.gd_error_string.restype = ctypes.c_char_p
        lib.gd_error_string.argtypes = [ci]
        lib.gd_renderer_create.restype = ci
        lib.gd_renderer_create.argtypes = [vp, vp, sz, ci, ci, ctypes.POINTER(vp)]
        lib.gd_renderer_destroy.restype = None
        lib.gd_renderer_destroy.argtypes = [vp]
        lib.gd_renderer_scratch_bytes.restype = sz
        lib.gd_renderer_scratch_bytes.argtypes = [vp]
        lib.gd_renderer_ctas.restype = ci
        lib.gd_renderer_ctas.argtypes = [vp]
        lib.gd_renderer_shared_bytes.restype = sz
        lib.gd_renderer_shared_bytes.argtypes = [vp]
        lib.gd_renderer_shared_bytes_view.restype = sz
        lib.gd_renderer_shared_bytes_view.argtypes = [vp]
        lib.gd_render_step.restype = ci
        lib.gd_render_step.argtypes = [vp, vp, vp, ci, ci, vp, vp, sz, vp, vp]
        lib.gd_render_reset.restype = ci
        lib.gd_render_reset.argtypes = [vp, vp, vp, ci, ci, vp, vp, vp, sz, vp, vp]
        lib.gd_render_frames.restype = ci
        lib.gd_render_frames.argtypes = [vp, vp, vp, ci, ci, ci, vp, vp, vp, vp, sz, vp, vp]
        lib.gd_render_step_frames.restype = ci
        lib.gd_render_step_frames.argtypes = [vp, vp, vp, ci, ci, ci, vp, vp, vp, vp, sz, vp, vp]
        lib.gd_render_step_ring.restype = ci
        lib.gd_render_step_ring.argtypes = [vp, vp, vp, ci, ci, vp, ci, vp, sz, vp, vp]
        lib.gd_render_reset_ring.restype = ci
        lib.gd_render_reset_ring.argtypes = [vp, vp, vp, ci, ci, vp, vp, vp, sz, vp, vp]
        lib.gd_render_step_host.restype = ci
        lib.gd_render_step_host.argtypes = [vp, vp, vp, ci, ci, vp, vp, vp, vp, vp, sz, vp, vp]
        lib.gd_static_scratch_bytes.restype = sz
        lib.gd_static_scratch_bytes.argtypes = []
        lib.gd_static_max_walls.restype = ci
        lib.gd_static_max_walls.argtypes = []
        lib.gd_render_step_static.restype = ci
        lib.gd_render_step_static.argtypes = [vp, vp, vp, ci, ci, vp, vp, vp]
        lib.gd_pack_state_scratch_bytes.restype = sz
        lib.gd_pack_state_scratch_bytes.argtypes = []
        lib.gd_pack_state.restype = ci
        lib.gd_pack_state.argtypes = [vp, vp, vp, vp, vp, sz, vp, vp]
        lib.gd_player_tics.restype = ci
        lib.gd_player_tics.argtypes = [vp, vp, vp, vp, ci, ci, ci, vp, vp, vp]
        lib.gd_renderer_bind_decals.restype = ci
        lib.gd_renderer_bind_decals.argtypes = [vp, vp, ci]
        lib.gd_probe_libm.restype = ci
        lib.gd_probe_libm.argtypes = [ci, vp, vp, vp, ci, vp]
        _libs[path] = lib
    return _libs[path]


def _check(code: int, what: str) -> None:
    if code != GD_OK:
        raise NativeError(f"{what} failed: {load().gd_error_string(code).decode()} ({code})")


def _ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


PROBE_ATAN2F, PROBE_COSF, PROBE_SINF, PROBE_HYPOT = 0, 1, 2, 3


def probe_libm(function: int, a: torch.Tensor, b: torch.Tensor | None = None) -> torch.Tensor:
    """The device's float32 ``atan2f(a, b)`` / ``cosf(a)`` / ``sinf(a)`` / ``sqrtf(a*a + b*b)`` as the
    kernels call them (diagnostic; see ``gd_probe_libm`` in the header)."""

    if a.dtype != torch.float32 or not a.is_cuda or not a.is_contiguous():
        raise ValueError("a must be a contiguous float32 CUDA tensor")
    if b is not None and (b.dtype != torch.float32 or b.shape != a.shape or b.device != a.device or not b.is_contiguous()):
        raise ValueError("b must match a")
    out = torch.empty_like(a)
    with torch.cuda.device(a.device):
        _check(load().gd_probe_libm(int(function), a.data_ptr(), _ptr(b), out.data_ptr(), a.numel(),
                                    torch.cuda.current_stream(a.device).cuda_stream), "gd_probe_libm")
    return out


class Renderer:
    """A scene blob resident on one CUDA device plus the launch scratch.

    ``lanes`` is ``(N,32) int32`` and ``things`` ``(N,max_things,4) int32`` on
    the same device (layout: include/gradoom_b200_layout.h).
    """

    def __init__(self, blob: np.ndarray, device: torch.device | str, max_things: int, *, checked: bool = False):
        self.lib = load(checked)
        self.checked = checked
        self.device = torch.device(device)
        if self.device.type != "cuda":
            raise NativeError("the renderer needs a CUDA device; there is no CPU path")
        if self.device.index is None:
            self.device = torch.device("cuda", torch.cuda.current_device())
        self.max_things = int(max_things)
        blob = np.ascontiguousarray(blob, dtype=np.uint8)
        self._blob_host = blob
        self.blob = torch.from_numpy(blob).to(self.device)
        handle = ctypes.c_void_p()
        index = self.device.index if self.device.index is not None else torch.cuda.current_device()
        _check(self.lib.gd_renderer_create(blob.ctypes.data, self.blob.data_ptr(), blob.size, index,
                                           self.max_things, ctypes.byref(handle)), "gd_renderer_create")
        self.handle = handle
        self.scratch_bytes = int(self.lib.gd_renderer_scratch_bytes(handle))
        # zero-initialised: the tail holds the kernel's lane queue, which every launch leaves at zero
        self.scratch = torch.zeros(self.scratch_bytes, dtype=torch.uint8, device=self.device)
        self.status = torch.zeros(4, dtype=torch.int32, device=self.device)   # word 0 is the status word
        self.flags_scratch = torch.zeros(int(self.lib.gd_pack_state_scratch_bytes()), dtype=torch.uint8,
                                         device=self.device)
        self.ctas = int(self.lib.gd_renderer_ctas(handle))
        self.shared_bytes = int(self.lib.gd_renderer_shared_bytes(handle))
        self.shared_bytes_view = int(self.lib.gd_renderer_shared_bytes_view(handle))   # observation-only calls
        self.launches = 0
        self._decals = None

    def bind_decals(self, decals: torch.Tensor | None) -> None:
        """The lanes' bullet-chip rings for every later render call: ``(N, slots, 4) int32`` on the
        renderer's device, each record a ``gd_decal`` (serial, wall | style << 16, along and z as
        float bits; ``state.decal_records`` builds it), or None to unbind.  The tensor is kept alive
        by the renderer; lane ``l`` of a render call reads ring ``l``."""

        if decals is None:
            _check(self.lib.gd_renderer_bind_decals(self.handle, None, 0), "gd_renderer_bind_decals")
            self._decals = None
            return
        if decals.dtype != torch.int32 or decals.dim() != 3 or decals.shape[2] != 4 or not decals.is_contiguous():
            raise ValueError("decals must be a contiguous (N, slots, 4) int32 tensor of gd_decal records")
        if decals.device != self.device:
            raise TypeError("the decal rings must live on the renderer's device")
        with torch.cuda.device(self.device):
            _check(self.lib.gd_renderer_bind_decals(self.handle, decals.data_ptr(), int(decals.shape[1])),
                   "gd_renderer_bind_decals")
        self._decals = decals

    def close(self) -> None:
        if getattr(self, "handle", None):
            self.lib.gd_renderer_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _stream(self) -> int:
        return torch.cuda.current_stream(self.device).cuda_stream

    def _inputs(self, lanes: torch.Tensor, things: torch.Tensor) -> int:
        if lanes.dtype != torch.int32 or lanes.dim() != 2 or lanes.shape[1] != 32 or not lanes.is_contiguous():
            raise ValueError("lanes must be a contiguous (N,32) int32 tensor")
        n = lanes.shape[0]
        if things.dtype != torch.int32 or tuple(things.shape) != (n, max(self.max_things, 1), 4) \
                or not things.is_contiguous():
            raise ValueError(f"things must be a contiguous (N,{max(self.max_things, 1)},4) int32 tensor")
        if lanes.device != self.device or things.device != self.device:
            raise TypeError("lanes and things must live on the renderer's device")
        if self._decals is not None and self._decals.shape[0] < n:
            raise ValueError(f"the bound decal rings cover {self._decals.shape[0]} lanes, the call draws {n}")
        return n

    def pack_state(self, engine_state, lanes, things):
        """Fill ``lanes`` / ``things`` from engine-shaped tensors on the device
        (``engine_state``: a ``state.EngineState``); two small launches on the
        current stream, no host synchronisation."""

        n = self._inputs(lanes, things)
        if engine_state.n != n:
            raise ValueError(f"the state has {engine_state.n} lanes, the record buffers {n}")
        if engine_state.device != self.device:
            raise TypeError("the state tensors must live on the renderer's device")
        with torch.cuda.device(self.device):
            _check(self.lib.gd_pack_state(self.handle, ctypes.byref(engine_state.struct), lanes.data_ptr(),
                                          things.data_ptr(), self.flags_scratch.data_ptr(),
                                          self.flags_scratch.numel(), self.status.data_ptr(), self._stream()),
                   "gd_pack_state")
        self.launches += 2

    def player_tics(self, players, buttons, tics, episode_timeout, *, lanes=None, actors=None):
        """Advance the player kinematics records ``players (N,24) int32`` in place by ``tics``
        game tics under ``buttons (N,) int32`` button masks; with ``lanes`` the new pose is
        also written into the lane records.  ``actors``: a ``state.SolidActors`` or None."""

        n = players.shape[0]
        if players.dtype != torch.int32 or players.dim() != 2 or players.shape[1] != 24 or not players.is_contiguous():
            raise ValueError("players must be a contiguous (N,24) int32 tensor")
        if buttons.dtype != torch.int32 or tuple(buttons.shape) != (n,) or not buttons.is_contiguous():
            raise ValueError("buttons must be a contiguous (N,) int32 tensor of button masks")
        if lanes is not None and (lanes.dtype != torch.int32 or tuple(lanes.shape) != (n, 32) or not lanes.is_contiguous()):
            raise ValueError("lanes must be a contiguous (N,32) int32 tensor")
        for t in (players, buttons, lanes):
            if t is not None and t.device != self.device:
                raise TypeError("the kinematics buffers must live on the renderer's device")
        with torch.cuda.device(self.device):
            _check(self.lib.gd_player_tics(self.handle, players.data_ptr(), buttons.data_ptr(),
                                           None if actors is None else ctypes.byref(actors.struct), n, int(tics),
                                           int(episode_timeout), _ptr(lanes), self.status.data_ptr(), self._stream()),
                   "gd_player_tics")
        self.launches += 1

    def step(self, lanes, things, stack, mask_hud=True):
        n = self._inputs(lanes, things)
        self._check_stack(stack, n)
        _check(self.lib.gd_render_step(self.handle, lanes.data_ptr(), things.data_ptr(), n, int(mask_hud),
                                       stack.data_ptr(), self.scratch.data_ptr(), self.scratch_bytes,
                                       self.status.data_ptr(), self._stream()), "gd_render_step")
        self.launches += 1

    def step_static(self, lanes, things, stack, mask_hud=True):
        """``step`` without any caller-provided scratch: for hosts that must not
        allocate device memory, the library's built-in scratch array is used
        (scenes up to ``gd_static_max_walls()`` walls; calls must not overlap)."""

        n = self._inputs(lanes, things)
        self._check_stack(stack, n)
        with torch.cuda.device(self.device):
            _check(self.lib.gd_render_step_static(self.handle, lanes.data_ptr(), things.data_ptr(), n,
                                                  int(mask_hud), stack.data_ptr(), self.status.data_ptr(),
                                                  self._stream()), "gd_render_step_static")
        self.launches += 1

    def step_host(self, lanes_host, things_host, lanes_dev, things_dev, stack, obs_host, mask_hud=True):
        """Host-buffer step: pinned ``lanes_host``/``things_host`` in, pinned
        ``obs_host (N,84,84) uint8`` out, all queued on the current stream."""

        n = self._inputs(lanes_dev, things_dev)
        self._check_stack(stack, n)
        for t in (lanes_host, things_host, obs_host):
            if t.device.type != "cpu" or not t.is_contiguous():
                raise TypeError("host buffers must be contiguous CPU tensors")
        if tuple(lanes_host.shape) != tuple(lanes_dev.shape) or tuple(things_host.shape) != tuple(things_dev.shape):
            raise ValueError("host and device record buffers must have the same shape")
        if tuple(obs_host.shape) != (n, 84, 84) or obs_host.dtype != torch.uint8:
            raise ValueError("obs_host must be (N,84,84) uint8")
        _check(self.lib.gd_render_step_host(self.handle, lanes_host.data_ptr(), things_host.data_ptr(), n,
                                            int(mask_hud), lanes_dev.data_ptr(), things_dev.data_ptr(),
                                            stack.data_ptr(), obs_host.data_ptr(), self.scratch.data_ptr(),
                                            self.scratch_bytes, self.status.data_ptr(), self._stream()),
               "gd_render_step_host")
        self.launches += 1

    def reset(self, lanes, things, reset_mask, stack, mask_hud=True):
        n = self._inputs(lanes, things)
        self._check_stack(stack, n)
        if reset_mask.dtype not in (torch.bool, torch.uint8) or tuple(reset_mask.shape) != (n,):
            raise TypeError("reset_mask must be a bool (N,) tensor")
        mask = reset_mask.contiguous().view(torch.uint8) if reset_mask.dtype == torch.bool else reset_mask
        mask16 = torch.zeros(((n + 15) // 16) * 16, dtype=torch.uint8, device=self.device)
        mask16[:n] = mask
        _check(self.lib.gd_render_reset(self.handle, lanes.data_ptr(), things.data_ptr(), n, int(mask_hud),
                                        mask16.data_ptr(), stack.data_ptr(), self.scratch.data_ptr(),
                                        self.scratch_bytes, self.status.data_ptr(), self._stream()),
               "gd_render_reset")
        self.launches += 1

    def frames(self, lanes, things, *, obs=False, indexed=False, rgb=False, mask_hud=True, include_hud=True):
        n = self._inputs(lanes, things)
        o = torch.empty((n, 84, 84), dtype=torch.uint8, device=self.device) if obs else None
        i = torch.empty((n, 240, 320), dtype=torch.uint8, device=self.device) if indexed else None
        c = torch.empty((n, 240, 320, 3), dtype=torch.uint8, device=self.device) if rgb else None
        _check(self.lib.gd_render_frames(self.handle, lanes.data_ptr(), things.data_ptr(), n, int(mask_hud),
                                         int(include_hud), _ptr(o), _ptr(i), _ptr(c), self.scratch.data_ptr(),
                                         self.scratch_bytes, self.status.data_ptr(), self._stream()),
               "gd_render_frames")
        self.launches += 1
        return o, i, c

    def step_frames(self, lanes, things, stack, *, indexed=None, rgb=None, mask_hud=True, include_hud=True):
        """One step (stack push) that also writes the full frame(s) of the same
        drawing pass into the caller's ``indexed (N,240,320)`` / ``rgb
        (N,240,320,3)`` uint8 tensors."""

        n = self._inputs(lanes, things)
        self._check_stack(stack, n)
        for t, shape in ((indexed, (n, 240, 320)), (rgb, (n, 240, 320, 3))):
            if t is not None and (t.dtype != torch.uint8 or tuple(t.shape) != shape or not t.is_contiguous()
                                  or t.device != self.device):
                raise ValueError(f"frame output must be a contiguous uint8 tensor of shape {shape} on the device")
        _check(self.lib.gd_render_step_frames(self.handle, lanes.data_ptr(), things.data_ptr(), n, int(mask_hud),
                                              int(include_hud), stack.data_ptr(), _ptr(indexed), _ptr(rgb),
                                              self.scratch.data_ptr(), self.scratch_bytes, self.status.data_ptr(),
                                              self._stream()), "gd_render_step_frames")
        self.launches += 1

    def _check_ring(self, ring, n):
        if ring.dtype != torch.uint8 or tuple(ring.shape) != (n, 8, 84, 84) or not ring.is_contiguous():
            raise ValueError("ring must be a contiguous (N,8,84,84) uint8 tensor")
        if ring.device != self.device:
            raise TypeError("ring must live on the renderer's device")

    def step_ring(self, lanes, things, ring, head, mask_hud=True):
        """One step on the mirrored ring: the new frame goes to slots ``head`` and
        ``head + 4``; ``ring[:, head + 1:head + 5]`` is then the four-frame window."""

        n = self._inputs(lanes, things)
        self._check_ring(ring, n)
        _check(self.lib.gd_render_step_ring(self.handle, lanes.data_ptr(), things.data_ptr(), n, int(mask_hud),
                                            ring.data_ptr(), int(head), self.scratch.data_ptr(), self.scratch_bytes,
                                            self.status.data_ptr(), self._stream()), "gd_render_step_ring")
        self.launches += 1

    def reset_ring(self, lanes, things, reset_mask, ring, mask_hud=True):
        n = self._inputs(lanes, things)
        self._check_ring(ring, n)
        if reset_mask.dtype not in (torch.bool, torch.uint8) or tuple(reset_mask.shape) != (n,):
            raise TypeError("reset_mask must be a bool (N,) tensor")
        mask = reset_mask.contiguous().view(torch.uint8) if reset_mask.dtype == torch.bool else reset_mask
        _check(self.lib.gd_render_reset_ring(self.handle, lanes.data_ptr(), things.data_ptr(), n, int(mask_hud),
                                             mask.data_ptr(), ring.data_ptr(), self.scratch.data_ptr(),
                                             self.scratch_bytes, self.status.data_ptr(), self._stream()),
               "gd_render_reset_ring")
        self.launches += 1

    def _check_stack(self, stack, n):
        if stack.dtype != torch.uint8 or tuple(stack.shape) != (n, 4, 84, 84) or not stack.is_contiguous():
            raise ValueError("stack must be a contiguous (N,4,84,84) uint8 tensor")
        if stack.device != self.device:
            raise TypeError("stack must live on the renderer's device")

    def check_status(self) -> None:
        """Synchronising read of the device status word; raises on any flag."""

        bits = int(self.status[0].item())
        if bits:
            self.status.zero_()
            names = []
            if bits & STATUS_EVENT_OVERFLOW:
                names.append("clip-event overflow (a column crossed more segs than the scratch holds)")
            if bits & STATUS_THINGS_OVERFLOW:
                names.append("a lane listed more things than max_things")
            if bits & STATUS_BAD_SECTOR:
                names.append("a sector index outside the scene (checked build)")
            if bits & STATUS_BAD_INDEX:
                names.append("a wall, texture, sprite or patch index outside its table (checked build)")
            if bits & STATUS_BAD_STATE:
                names.append("a lane or thing record with a value outside its range (checked build)")
            raise NativeError("renderer status: " + "; ".join(names or [hex(bits)]))
