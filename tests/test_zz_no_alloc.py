"""The allocation-free entry point, `gd_render_step_static`.

Some hosts of this library are not allowed to allocate GPU memory (a plugin in
a process whose memory pool belongs to the embedding application, or code that
runs after the allocator was frozen), so they cannot hand the renderer its
scratch buffer.  For them the library carries a fixed scratch array.  This test
calls that entry point through the C ABI twice in a row and requires the frame
stacks to equal, byte for byte, what the regular entry point produces from the
same inputs; the second call checks that nothing stale is left in the shared
array by the first.  It is collected last so that a failure here cannot hide
any other test.
"""

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


def test_static_scratch_step_matches_regular_step(pkg, scenes):
    from gradoom_b200 import native, stepper

    sc, blob = scenes("c2")
    n, k = 200, 12
    renderer = native.Renderer(blob, DEV, k)
    lib = native.load()
    assert sc.num_walls <= lib.gd_static_max_walls()
    assert 0 < lib.gd_static_scratch_bytes() < 32 << 20
    rng = np.random.default_rng(4)
    start = torch.from_numpy(rng.integers(0, 256, size=(n, 4, 84, 84), dtype=np.uint8)).to(DEV)
    regular, static = start.clone(), start.clone()
    lanes, things = stepper.random_lanes(sc, n, k, seed=31)
    stream = torch.cuda.current_stream().cuda_stream
    for call in range(2):
        dl, dt = torch.from_numpy(lanes).to(DEV), torch.from_numpy(things).to(DEV)
        renderer.step(dl, dt, regular)
        rc = lib.gd_render_step_static(renderer.handle, dl.data_ptr(), dt.data_ptr(), n, 1, static.data_ptr(),
                                       renderer.status.data_ptr(), stream)
        assert rc == 0, lib.gd_error_string(rc)
        torch.cuda.synchronize()
        renderer.check_status()
        assert torch.equal(static, regular), f"call {call}"
        stepper.advance(sc, lanes, seed=call)
    assert not torch.equal(static, start)


def test_static_scratch_rejects_scenes_beyond_its_limit(pkg, scenes):
    from gradoom_b200 import native, stepper

    sc, blob = scenes("c4")          # 800 walls: more than the built-in array is sized for
    renderer = native.Renderer(blob, DEV, 4)
    lib = native.load()
    assert sc.num_walls > lib.gd_static_max_walls()
    lanes, things = stepper.random_lanes(sc, 2, 4, seed=1)
    dl, dt = torch.from_numpy(lanes).to(DEV), torch.from_numpy(things).to(DEV)
    stack = torch.zeros((2, 4, 84, 84), dtype=torch.uint8, device=DEV)
    rc = lib.gd_render_step_static(renderer.handle, dl.data_ptr(), dt.data_ptr(), 2, 1, stack.data_ptr(),
                                   renderer.status.data_ptr(), torch.cuda.current_stream().cuda_stream)
    assert rc == -9
    assert b"built-in scratch" in lib.gd_error_string(rc)
    assert int(stack.max()) == 0
