"""retention.AUTO_CHUNK: a request for a small chunk runs with a larger one; everything the caller sees - padding,
outputs, gradients, the state after the last token - is that of the request."""
import pytest
import torch
import torch.nn.functional as F

from tests._golden import rel_l2


def test_effective_chunk_table():
    from retention_integration_b200 import retention

    retention.AUTO_CHUNK = True
    want = {(65536, 128): 1024, (2000, 128): 1024, (1152, 128): 384, (512, 128): 512, (31, 128): 128, (4096, 256): 1024,
            (65536, 1024): 1024, (300, None): None, (768, 192): 768, (5000, 64): 1024,
            # above the fast size: a divisor of the request; no chunking asked for: chunked when the sequence is long
            (65536, 2048): 1024, (65536, 4096): 1024, (5000, 1536): 768, (1000, 3000): 1000, (4096, 1031): 1031,
            (3000, None): 1024, (70000, None): 1024, (2100, None): None, (500, None): None}
    for (t, c), ce in want.items():
        assert retention.effective_chunk(t, c) == ce, (t, c)
        if c is not None and c < 1024:
            assert ce % c == 0 and -(-t // ce) * ce <= (-(-t // c) * c) * 17 // 16
        if c is not None and c > 1024:
            assert c % ce == 0
    assert retention.effective_chunk(65536, None, deg=4) is None  # deg 4 forms no states
    retention.AUTO_CHUNK = False
    assert retention.effective_chunk(65536, 128) == 128 and retention.effective_chunk(65536, None) is None


@pytest.mark.gpu
@pytest.mark.parametrize("t,c,r,states", [(2000, 128, 1, False), (1152, 128, 2, True), (4096, 256, 1, True),
                                          (3000, None, 1, False), (4000, 2048, 1, True), (3000, 3000, 2, False)])
def test_auto_chunk_gives_the_requested_chunks_results(cuda_device, t, c, r, states):
    import retention_integration_b200 as prb
    from retention_integration_b200 import retention

    g = torch.Generator().manual_seed(t + (c or 0))
    b, h, d = 2, 2, 64
    Q = torch.randn(b, t, h * r, d, generator=g).bfloat16().to(cuda_device)
    K, V = (torch.randn(b, t, h, d, generator=g).bfloat16().to(cuda_device) for _ in range(2))
    lg = F.logsigmoid(torch.randn(b, t, h, generator=g) + 2.0).to(cuda_device)
    dO = torch.randn(b, t, h * r, d, generator=g).bfloat16().to(cuda_device)

    def run(auto):
        retention.AUTO_CHUNK = auto
        leaves = [x.clone().requires_grad_(True) for x in (Q, K, V, lg)]
        out = prb.power_retention(*leaves, deg=2, chunk_size=c, return_final_state=states)
        O, final = out if states else (out, None)
        O.backward(dO)
        return [O] + [x.grad for x in leaves] + (list(final) if states else [])

    asked, auto = run(False), run(True)
    assert retention.effective_chunk(t, c) != c
    for a, bb in zip(asked, auto):
        assert a.shape == bb.shape
        assert rel_l2(bb.float(), a.float()) < 6e-3


@pytest.mark.gpu
def test_auto_chunk_with_a_carried_state(cuda_device):
    """Two segments chained through initial_state / return_final_state, each run with its own automatic chunk
    (1024 for the first, 640 for the second), against the same chain at the requested chunk of 128."""
    import retention_integration_b200 as prb
    from retention_integration_b200 import retention

    g = torch.Generator().manual_seed(77)
    b, h, d, t1, t2 = 1, 2, 64, 1024, 1280
    Q = torch.randn(b, t1 + t2, h, d, generator=g).bfloat16().to(cuda_device)
    K, V = (torch.randn(b, t1 + t2, h, d, generator=g).bfloat16().to(cuda_device) for _ in range(2))
    lg = F.logsigmoid(torch.randn(b, t1 + t2, h, generator=g) + 3.0).to(cuda_device)

    def chain(auto):
        retention.AUTO_CHUNK = auto
        with torch.no_grad():
            o1, st = prb.power_retention(Q[:, :t1], K[:, :t1], V[:, :t1], lg[:, :t1], chunk_size=128,
                                         return_final_state=True)
            o2, st2 = prb.power_retention(Q[:, t1:], K[:, t1:], V[:, t1:], lg[:, t1:], chunk_size=128, initial_state=st,
                                          return_final_state=True)
        return torch.cat([o1, o2], 1), st2

    (o_a, st_a), (o_b, st_b) = chain(False), chain(True)
    assert retention.effective_chunk(t1, 128) == 1024 and retention.effective_chunk(t2, 128) == 640
    assert rel_l2(o_b.float(), o_a.float()) < 6e-3
    assert rel_l2(st_b[0].float(), st_a[0].float()) < 6e-3 and rel_l2(st_b[1], st_a[1]) < 1e-3


def test_c_abi_helper_agrees_with_the_python_choice():
    """pr_fast_chunk is pure host arithmetic: callable without a GPU."""
    import ctypes

    from retention_integration_b200 import _lib, retention

    retention.AUTO_CHUNK = True
    fn = _lib.lib().pr_fast_chunk
    fn.argtypes, fn.restype = [ctypes.c_longlong, ctypes.c_int], ctypes.c_int
    for t in (17, 500, 1000, 1152, 2000, 2100, 3000, 4096, 5000, 65536, 70000):
        for c in (None, 64, 96, 128, 192, 256, 320, 512, 1024, 1031, 1536, 2048, 3000, 4096):
            assert fn(t, c or 0) == (retention.effective_chunk(t, c) or 0), (t, c)


def test_effective_chunk_properties():
    """Whatever is asked for: the chosen chunk is a multiple of a small request (a divisor of a large one), never
    above 1024 unless the request itself has no divisor there, pads by at most 1/16 more, and the C helper agrees."""
    import ctypes
    import random

    from retention_integration_b200 import _lib, retention

    retention.AUTO_CHUNK = True
    fn = _lib.lib().pr_fast_chunk
    fn.argtypes, fn.restype = [ctypes.c_longlong, ctypes.c_int], ctypes.c_int
    rng = random.Random(0)
    for _ in range(3000):
        t = rng.randint(1, 300000)
        c = rng.choice([None, rng.randint(1, 1023), rng.randint(1025, 9000), 16 * rng.randint(1, 512)])
        ce = retention.effective_chunk(t, c)
        assert fn(t, c or 0) == (ce or 0)
        pad = lambda x: -(-t // x) * x
        if c is None:
            assert ce in (None, 512, 1024) and (ce is None or (t > 2048 and pad(ce) <= t + t // 16))
        elif c < 1024:
            assert ce % c == 0 and c <= ce <= 1024 and pad(ce) <= pad(c) + pad(c) // 16
        elif c > 1024:
            assert c % ce == 0 and (256 <= ce <= 1024 or ce == c) and pad(ce) <= pad(c)
        else:
            assert ce == c
