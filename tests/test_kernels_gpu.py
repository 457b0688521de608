"""Each kernel alone against a plain float32/float64 torch computation, at sizes other than the
tiny models': widths and vocabularies that are no power of two, odd head counts, head sizes in
steps of 16 (and one that is not), long and short rows."""
import math

import numpy as np
import pytest
import torch

import plain_falcon as plain

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]


def tol(dtype):
    return dict(atol=2e-5, rtol=1e-5) if dtype == torch.float32 else dict(atol=2e-2, rtol=2e-2)


@pytest.fixture(scope="module")
def K():
    from pytorch_transformers_b200 import kernels
    kernels.lib()
    return kernels


def rnd(*shape, dtype=torch.float32, scale=1.0, seed=0):
    g = torch.Generator().manual_seed(seed + sum(shape))
    return (torch.randn(*shape, generator=g) * scale).to(dtype).cuda()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("width", [7, 96, 1000, 4544])
def test_gather_rows(K, dtype, width):
    table = rnd(333, width, dtype=dtype)
    ids = torch.tensor([0, 332, 5, 5, 17], dtype=torch.int32).cuda()
    status = torch.zeros(1, dtype=torch.int32).cuda()
    out = K.gather_rows(ids, table, status)
    assert torch.equal(out, table[ids.long()])
    assert status.item() == 0
    bad = torch.tensor([1, 400], dtype=torch.int32).cuda()
    K.gather_rows(bad, table, status)
    assert status.item() == 1


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rows,width,eps", [(1, 64, 1e-5), (5, 96, 1e-6), (3, 4544, 1e-5), (2, 8192, 1e-5),
                                            (4, 1001, 1e-3), (2, 20000, 1e-5), (300, 4544, 1e-5), (2, 16384, 1e-5),
                                            (2, 16392, 1e-5), (7, 2056, 1e-5)])
def test_layernorm_and_pair(K, dtype, rows, width, eps):
    x = rnd(rows, width, dtype=dtype, scale=3.0) + 0.5
    g1, b1 = rnd(width, seed=1) + 1, rnd(width, seed=2)
    g2, b2 = rnd(width, seed=3) + 1, rnd(width, seed=4)
    ref1 = plain.layer_norm(x.double().cpu(), g1.double().cpu(), b1.double().cpu(), eps)
    ref2 = plain.layer_norm(x.double().cpu(), g2.double().cpu(), b2.double().cpu(), eps)
    y = K.norm(x, g1, b1, eps)
    torch.testing.assert_close(y.double().cpu(), ref1, **tol(dtype))
    y1, y2 = K.norm(x, g1, b1, eps, gain2=g2, bias2=b2)
    assert torch.equal(y1, y)
    torch.testing.assert_close(y2.double().cpu(), ref2, **tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
def test_rmsnorm(K, dtype):
    x = rnd(6, 200, dtype=dtype, scale=2.0)
    g = rnd(200, seed=1) + 1
    xd = x.double().cpu()
    ref = xd / torch.sqrt((xd ** 2).mean(-1, keepdim=True) + 1e-6) * g.double().cpu()
    torch.testing.assert_close(K.norm(x, g, None, 1e-6, "rmsnorm").double().cpu(), ref, **tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("act", ["none", "gelu", "gelu_new", "relu"])
def test_bias_act(K, dtype, act):
    y = rnd(9, 333, dtype=dtype, scale=2.0)
    b = rnd(333, seed=5)
    ref = y.double().cpu() + b.double().cpu()
    ref = ref if act == "none" else plain.activation(ref, act)
    out = K.bias_act_(y.clone(), b, act)
    torch.testing.assert_close(out.double().cpu(), ref, **tol(dtype))
    out2 = K.bias_act_(y.clone(), None, act)
    ref2 = y.double().cpu() if act == "none" else plain.activation(y.double().cpu(), act)
    torch.testing.assert_close(out2.double().cpu(), ref2, **tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
def test_residual(K, dtype):
    x, a, b = (rnd(11, 97, dtype=dtype, seed=s) for s in (1, 2, 3))
    ref = x.double() + (a.double() + b.double())
    torch.testing.assert_close(K.residual(x, a, b).double(), ref, **tol(dtype))
    torch.testing.assert_close(K.residual(x, a).double(), x.double() + a.double(), **tol(dtype))
    if dtype == torch.bfloat16:
        # one rounding of the float32 sum, not a rounding per addition
        exact = (x.float() + (a.float() + b.float())).bfloat16()
        assert torch.equal(K.residual(x, a, b), exact)


@pytest.mark.parametrize("m,n,k", [(1, 64, 64), (37, 101, 53), (64, 64, 16), (130, 4672 // 8, 71), (5, 1000, 96),
                                   (2, 65, 4544)])
@pytest.mark.parametrize("act,bias", [("none", False), ("gelu", True), ("none", True)])
def test_linear_f32(K, m, n, k, act, bias):
    x, w = rnd(m, k, seed=1), rnd(n, k, seed=2, scale=0.1)
    b = rnd(n, seed=3) if bias else None
    ref = x.double().cpu() @ w.double().cpu().T
    if bias:
        ref = ref + b.double().cpu()
    if act != "none":
        ref = plain.activation(ref, act)
    out = K.linear_f32(x, w, b, act)
    torch.testing.assert_close(out.double().cpu(), ref, atol=1e-5, rtol=1e-5)


def test_linear_f32_rows_do_not_depend_on_the_batch(K):
    x, w = rnd(70, 300, seed=1), rnd(129, 300, seed=2)
    full = K.linear_f32(x, w)
    for rows in ([0], [3, 4], list(range(65, 70))):
        part = K.linear_f32(x[rows].contiguous(), w)
        assert torch.equal(part, full[rows])


def test_to_float(K):
    x = rnd(3, 1000, dtype=torch.bfloat16)
    assert torch.equal(K.to_float(x), x.float())


@pytest.mark.parametrize("m", [1, 5, 8, 9, 16, 17, 32])
@pytest.mark.parametrize("n,k", [(100, 64), (4672, 4544), (71, 96), (1000, 18176 // 4)])
@pytest.mark.parametrize("act,bias,add,f32", [("none", False, False, False), ("gelu", True, False, False),
                                               ("none", True, True, False), ("none", False, False, True),
                                               ("relu", False, True, True)])
def test_skinny_linear(K, m, n, k, act, bias, add, f32):
    bf = torch.bfloat16
    x, w = rnd(m, k, dtype=bf, seed=1), rnd(n, k, dtype=bf, seed=2, scale=0.05)
    b = rnd(n, seed=3) if bias else None
    a = rnd(m, n, dtype=bf, seed=4) if add else None
    assert K.skinny_linear_takes(m, k)
    ref = x.double().cpu() @ w.double().cpu().T
    if bias:
        ref = ref + b.double().cpu()
    if act != "none":
        ref = plain.activation(ref, act)
    if add:
        ref = ref + a.double().cpu()
    out = K.skinny_linear(x, w, b, act, a, out_dtype=torch.float32 if f32 else bf)
    assert out.dtype == (torch.float32 if f32 else bf)
    if f32:
        torch.testing.assert_close(out.double().cpu(), ref, atol=1e-3, rtol=1e-4)
    else:
        torch.testing.assert_close(out.double().cpu(), ref, **tol(bf))


@pytest.mark.parametrize("m", [1, 7, 16, 17, 33, 64, 100, 128])
@pytest.mark.parametrize("n,k", [(100, 64), (4672, 4544), (71, 96), (18176 // 2, 4544), (333, 18176 // 4),
                                 (4544, 1160), (129, 1024), (128, 8)])
@pytest.mark.parametrize("act,bias,add,f32", [("none", False, False, False), ("gelu", True, False, False),
                                               ("none", True, True, False), ("relu", False, True, True)])
def test_tc_linear(K, m, n, k, act, bias, add, f32):
    """The tcgen05 linear layer: every number of rows up to 128, widths that are no multiple of the
    128-row tile or of the 64-wide k chunk, with and without the division of K over a cluster."""
    bf = torch.bfloat16
    x, w = rnd(m, k, dtype=bf, seed=1), rnd(n, k, dtype=bf, seed=2, scale=0.05)
    b = rnd(n, seed=3) if bias else None
    a = rnd(m, n, dtype=bf, seed=4) if add else None
    assert K.tc_linear_takes(m, k)
    ref = x.double().cpu() @ w.double().cpu().T
    if bias:
        ref = ref + b.double().cpu()
    if act != "none":
        ref = plain.activation(ref, act)
    if add:
        ref = ref + a.double().cpu()
    out = K.tc_linear(x, w, b, act, a, out_dtype=torch.float32 if f32 else bf)
    K.check_device_errors(x.device)
    assert out.dtype == (torch.float32 if f32 else bf)
    if f32:
        torch.testing.assert_close(out.double().cpu(), ref, atol=1e-3, rtol=1e-4)
    else:
        torch.testing.assert_close(out.double().cpu(), ref, **tol(bf))


def test_tc_linear_one_key_stands_out(K):
    """A single large product far along K, in a block's last chunk, must arrive in the sum: one weight
    row and one token get a matching spike at the last k."""
    bf = torch.bfloat16
    m, n, k = 48, 4544, 4544
    x, w = rnd(m, k, dtype=bf, seed=1, scale=0.01), rnd(n, k, dtype=bf, seed=2, scale=0.01)
    x[37, k - 1] = 8.0
    w[4001, k - 1] = 4.0
    out = K.tc_linear(x, w).float().cpu()
    K.check_device_errors(x.device)
    ref = (x.double().cpu() @ w.double().cpu().T).float()
    assert abs(out[37, 4001] - 32.0) < 0.5
    torch.testing.assert_close(out, ref, **tol(bf))


def test_tc_linear_refuses_what_it_does_not_take(K):
    from pytorch_transformers_b200.kernels import KernelError
    assert K.lib().ptb_tc_linear_max_rows() == K.TC_LINEAR_MAX_ROWS
    assert K.lib().ptb_tc_linear_k_multiple() == K.TC_LINEAR_K_MULTIPLE
    assert not K.tc_linear_takes(129, 64) and not K.tc_linear_takes(4, 36)
    bf = torch.bfloat16
    with pytest.raises(KernelError):
        K.tc_linear(rnd(129, 64, dtype=bf), rnd(16, 64, dtype=bf))
    with pytest.raises(KernelError):
        K.tc_linear(rnd(4, 36, dtype=bf), rnd(16, 36, dtype=bf))
    with pytest.raises(KernelError):
        K.tc_linear(rnd(4, 64), rnd(16, 64))


@pytest.mark.parametrize("m", [1, 8, 16])
@pytest.mark.parametrize("n,k,shares", [(8192, 32768, 2), (4096, 65568, 4)])
def test_skinny_linear_k_divided_among_blocks(K, m, n, k, shares):
    """512 and 256 tiles of 16 rows do not divide evenly over 148 SMs and K is long enough: 2 and 4 blocks
    per tile, partial sums through scratch memory, the last block by ticket runs the epilogue. Twice in a
    row: the tickets must be back at zero. The second K leaves a ragged last round."""
    bf = torch.bfloat16
    assert K._skinny_scratch_floats(m, n, k) == (n // 16) * shares * 16 * (8 if m <= 8 else 16)
    assert K._skinny_scratch_floats(m, 4544, 18176) == 0
    x, w = rnd(m, k, dtype=bf, seed=1, scale=0.3), rnd(n, k, dtype=bf, seed=2, scale=0.05)
    b, a = rnd(n, seed=3), rnd(m, n, dtype=bf, seed=4)
    ref = plain.activation(x.double().cpu() @ w.double().cpu().T + b.double().cpu(), "gelu") + a.double().cpu()
    for _ in range(2):
        out = K.skinny_linear(x, w, b, "gelu", a)
        torch.testing.assert_close(out.double().cpu(), ref, **tol(bf))
    assert int(K._ticket_arenas[x.device][0].abs().sum()) == 0


def test_two_divided_launches_at_the_same_time_do_not_share_their_tickets(K):
    """Two launches that divide K among blocks run side by side on two streams (as the two branches of a
    block do inside a step): each counts its blocks' arrivals in words of its own, so both give what
    they give alone. Tickets never wait for anybody, so a fault here shows as a wrong sum, not a hang."""
    bf = torch.bfloat16
    m, n, k = 8, 8192, 32768
    assert K._skinny_scratch_floats(m, n, k) > 0
    xs = [rnd(m, k, dtype=bf, seed=s, scale=0.3) for s in (1, 2)]
    ws = [rnd(n, k, dtype=bf, seed=s, scale=0.05) for s in (3, 4)]
    alone = [K.skinny_linear(x, w) for x, w in zip(xs, ws)]
    torch.cuda.synchronize()
    streams = [torch.cuda.Stream(), torch.cuda.Stream()]
    for _ in range(10):
        outs = []
        for st, x, w in zip(streams, xs, ws):
            st.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(st):
                outs.append([K.skinny_linear(x, w) for _ in range(3)])
        for st in streams:
            torch.cuda.current_stream().wait_stream(st)
        torch.cuda.synchronize()
        for got, want in zip(outs, alone):
            for g in got:
                assert torch.equal(g, want)
    assert int(K._ticket_arenas[xs[0].device][0].abs().sum()) == 0
    # a launch's words are its own: consecutive launches get consecutive stretches of the arena
    a, b = K._tickets(100, xs[0].device), K._tickets(100, xs[0].device)
    assert a.data_ptr() != b.data_ptr() and a.numel() == 128


def test_skinny_linear_refuses_what_it_does_not_take(K):
    from pytorch_transformers_b200.kernels import KernelError
    assert K.lib().ptb_skinny_linear_max_rows() == K.SKINNY_MAX_ROWS
    assert K.lib().ptb_skinny_linear_k_multiple() == K.SKINNY_K_MULTIPLE
    assert not K.skinny_linear_takes(33, 64) and not K.skinny_linear_takes(4, 48)
    with pytest.raises(KernelError):
        K.skinny_linear(rnd(33, 64, dtype=torch.bfloat16), rnd(16, 64, dtype=torch.bfloat16))
    with pytest.raises(KernelError):
        K.skinny_linear(rnd(4, 48, dtype=torch.bfloat16), rnd(16, 48, dtype=torch.bfloat16))
    with pytest.raises(KernelError):
        K.skinny_linear(rnd(4, 64), rnd(16, 64))




def test_a_bounded_wait_that_runs_out_raises_on_the_host_and_leaves_the_device_usable(K):
    """Every wait on an mbarrier in the tcgen05 kernels gives up after a number of tries, raises a flag
    in device memory and lets the kernel return. Here a kernel waits 1,000 tries on a barrier at which
    nobody arrives (no fault, no hang: the wait simply runs out); the host's check then raises once,
    the flag is clean again afterwards, and a tcgen05 kernel still runs."""
    from pytorch_transformers_b200.kernels import KernelError
    dev = torch.device("cuda", torch.cuda.current_device())
    K.check_device_errors(dev)                           # clean before
    gave_up = K.selftest_bounded_wait(dev, tries=1000)
    with pytest.raises(KernelError, match="gave up waiting .*code 99"):
        K.check_device_errors(dev)
    assert int(gave_up.item()) == 1
    K.check_device_errors(dev)                           # raised once, clean again
    bf = torch.bfloat16
    x, w = rnd(40, 256, dtype=bf, seed=1), rnd(300, 256, dtype=bf, seed=2, scale=0.05)
    out = K.tc_linear(x, w)
    K.check_device_errors(dev)
    torch.testing.assert_close(out.double().cpu(), x.double().cpu() @ w.double().cpu().T, **tol(bf))
    with pytest.raises(KernelError):
        K.selftest_bounded_wait(dev, tries=0)
