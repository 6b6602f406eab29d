"""The general pointwise loops (broadcast, strided views, type promotion, Scalars, every element type) against the
CPU results of the same expressions, and a check that none of them took the library fallback.
Parity: reference tests/unittest/operator/test_{binary,unary,compare,where,clamp}.py (CPU-oracle comparisons)."""
import pytest
import torch

pytestmark = pytest.mark.gpu

FLOATS = [torch.float32, torch.bfloat16, torch.float16, torch.float64]
INTS = [torch.int32, torch.int64, torch.uint8, torch.int8, torch.int16]


def _rand(shape, dt, positive=False):
    g = torch.Generator().manual_seed(hash((tuple(shape), str(dt))) % (1 << 31))
    if dt.is_floating_point:
        t = torch.randn(shape, generator=g)
        if positive:
            t = t.abs() + 0.5
        return t.to(dt)
    if dt == torch.bool:
        return torch.rand(shape, generator=g) > 0.5
    lo = 1 if positive else (0 if dt == torch.uint8 else -20)
    return torch.randint(lo, 20, shape, generator=g).to(dt)


def _check(fn, inputs, dev, tol=None):
    ref = fn(*inputs)
    out = fn(*[x.to(dev) if isinstance(x, torch.Tensor) else x for x in inputs])
    assert out.dtype == ref.dtype, (out.dtype, ref.dtype)
    assert out.shape == ref.shape
    if ref.dtype.is_floating_point:
        t = tol or {torch.float32: 1e-5, torch.float64: 1e-10, torch.bfloat16: 2e-2, torch.float16: 4e-3}[ref.dtype]
        assert torch.allclose(out.cpu().double(), ref.double(), atol=t, rtol=t, equal_nan=True), \
            (out.cpu().double() - ref.double()).abs().max()
    else:
        assert torch.equal(out.cpu(), ref)


BINARY = {
    "add": torch.add, "sub": torch.sub, "mul": torch.mul, "maximum": torch.maximum, "minimum": torch.minimum,
    "eq": torch.eq, "ne": torch.ne, "lt": torch.lt, "le": torch.le, "gt": torch.gt, "ge": torch.ge,
}


@pytest.mark.parametrize("name", sorted(BINARY))
@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16, torch.int64, torch.int32, torch.uint8])
def test_binary_broadcast(bw, dev, name, dt):
    bw.reset_fallback_counts()
    fn = BINARY[name]
    _check(fn, (_rand((4, 1, 33), dt), _rand((5, 33), dt)), dev)           # broadcast both ways
    _check(fn, (_rand((7, 9), dt).t(), _rand((9, 7), dt)), dev)            # a transposed view
    _check(fn, (_rand((3, 8), dt)[:, ::2], _rand((4,), dt)), dev)          # strided + broadcast
    if name not in ("maximum", "minimum"):
        _check(fn, (_rand((6, 5), dt), 3), dev)                            # Python scalar
    assert not any(name in k for k in bw.fallback_counts()), bw.fallback_counts()


def test_type_promotion_and_division(bw, dev):
    bw.reset_fallback_counts()
    a_i, b_f = _rand((5, 6), torch.int64), _rand((6,), torch.float32)
    _check(torch.add, (a_i, b_f), dev)                                     # int + float -> float
    _check(torch.mul, (a_i, 2.5), dev)                                     # int * float scalar -> float
    _check(torch.mul, (_rand((4, 4), torch.bfloat16), _rand((4, 4), torch.float32)), dev)
    _check(torch.div, (a_i, _rand((5, 6), torch.int64, positive=True)), dev)          # true division of ints
    for mode in ("floor", "trunc"):
        _check(lambda x, y, m=mode: torch.div(x, y, rounding_mode=m), (a_i, _rand((6,), torch.int64, positive=True)), dev)
        _check(lambda x, y, m=mode: torch.div(x, y, rounding_mode=m), (_rand((5, 6), torch.float32), b_f), dev)
    _check(torch.remainder, (a_i, _rand((6,), torch.int64, positive=True)), dev)
    _check(torch.remainder, (_rand((5, 6), torch.float32), _rand((6,), torch.float32, positive=True)), dev)
    _check(torch.fmod, (_rand((5, 6), torch.float32), 1.5), dev)
    _check(torch.pow, (_rand((5, 6), torch.float32, positive=True), _rand((6,), torch.float32)), dev, tol=1e-4)
    _check(torch.pow, (_rand((5, 6), torch.float32), 2), dev)
    _check(torch.pow, (_rand((5, 6), torch.int64), 3), dev)
    _check(lambda e: torch.pow(2.0, e), (_rand((5, 6), torch.float32),), dev, tol=1e-5)
    _check(torch.atan2, (_rand((5, 6), torch.float32), _rand((6,), torch.float32)), dev)
    _check(torch.floor_divide, (a_i, _rand((6,), torch.int64, positive=True)), dev)
    _check(torch.bitwise_and, (_rand((5, 6), torch.int32), _rand((6,), torch.int32)), dev)
    _check(torch.bitwise_or, (_rand((5, 6), torch.bool), _rand((6,), torch.bool)), dev)
    _check(torch.bitwise_xor, (_rand((5, 6), torch.int64), 5), dev)
    _check(torch.logical_and, (_rand((5, 6), torch.float32), _rand((6,), torch.int64)), dev)
    _check(torch.logical_or, (_rand((5, 6), torch.bool), _rand((6,), torch.bool)), dev)
    _check(torch.logical_xor, (_rand((5, 6), torch.int32), _rand((6,), torch.int32)), dev)
    assert not bw.fallback_counts(), bw.fallback_counts()


UNARY_F = ["floor", "ceil", "round", "trunc", "frac", "sign", "exp2", "expm1", "sin", "cos", "tan", "erf", "exp", "tanh",
           "sigmoid", "neg", "abs", "isnan", "atan", "sinh", "cosh", "asinh", "erfc"]
UNARY_POS = ["log", "log2", "log10", "log1p", "sqrt", "rsqrt", "reciprocal"]


@pytest.mark.parametrize("dt", FLOATS)
def test_unary_float(bw, dev, dt):
    bw.reset_fallback_counts()
    for name in UNARY_F:
        _check(getattr(torch, name), (_rand((5, 7), dt).t(),), dev)        # non-contiguous: the general loop
        _check(getattr(torch, name), (_rand((64,), dt),), dev)             # dense: the fast path or the loop
    for name in UNARY_POS:
        _check(getattr(torch, name), (_rand((5, 7), dt, positive=True)[:, ::2],), dev)
    x = _rand((6, 6), dt)
    for name in ("asin", "acos", "atanh"):                                # domain (-1, 1)
        _check(lambda t, f=getattr(torch, name): f(t.clamp(-0.9, 0.9)), (x,), dev)
    _check(lambda t: torch.acosh(t.abs() + 1.25), (x,), dev)              # domain [1, inf)
    _check(lambda t: torch.nn.functional.gelu(t.t()), (x,), dev)
    _check(lambda t: torch.nn.functional.leaky_relu(t, 0.1), (x,), dev)
    _check(lambda t: torch.nn.functional.elu(t), (x,), dev)
    _check(lambda t: torch.nn.functional.softplus(t), (x,), dev)
    _check(lambda t: torch.nn.functional.hardtanh(t, -0.5, 0.5), (x,), dev)
    assert not bw.fallback_counts(), bw.fallback_counts()


def test_unary_integer_and_bool(bw, dev):
    bw.reset_fallback_counts()
    for dt in INTS:
        x = _rand((4, 9), dt)
        for name in ("abs", "neg", "sign") if dt != torch.uint8 else ("sign",):
            _check(getattr(torch, name), (x,), dev)
        _check(torch.bitwise_not, (x,), dev)
        _check(torch.logical_not, (x,), dev)
        _check(torch.exp, (x.clamp(-3, 3),), dev)                          # integer input, floating result
        _check(torch.sqrt, (x.abs(),), dev)
    _check(torch.logical_not, (_rand((4, 9), torch.bool),), dev)
    assert not bw.fallback_counts(), bw.fallback_counts()


def test_where_clamp_masked_fill_addc_lerp(bw, dev):
    bw.reset_fallback_counts()
    for dt in (torch.float32, torch.bfloat16, torch.int64):
        a, b = _rand((4, 1, 6), dt), _rand((5, 6), dt)
        cond = _rand((4, 5, 1), torch.bool)
        _check(torch.where, (cond, a, b), dev)
        _check(lambda c, x: torch.where(c, x, 0), (cond, a), dev)
        _check(lambda x: x.clamp(-1, 1), (b,), dev)
        _check(lambda x: x.clamp(min=0), (b,), dev)
        _check(lambda x: x.clamp(max=1), (b,), dev)
        _check(lambda x, m: x.masked_fill(m, 7), (b, _rand((5, 6), torch.bool)), dev)
        _check(lambda x, m: x.masked_fill(m, 7), (a.expand(4, 5, 6).contiguous(), cond), dev)   # broadcast mask
    x, t1, t2 = (_rand((5, 6), torch.float32) for _ in range(3))
    t2 = t2.abs() + 1
    _check(lambda a, b, c: torch.addcmul(a, b, c, value=0.5), (x, t1, t2), dev)
    _check(lambda a, b, c: torch.addcdiv(a, b, c, value=0.5), (x, t1, t2), dev)
    _check(lambda a, b: torch.lerp(a, b, 0.3), (x, t1), dev)
    _check(lambda a, b, w: torch.lerp(a, b, w), (x, t1, torch.rand(6)), dev)
    assert not bw.fallback_counts(), bw.fallback_counts()


def test_inplace_and_out_variants(bw, dev):
    bw.reset_fallback_counts()
    a, b = _rand((4, 6), torch.float32), _rand((6,), torch.float32)
    d = a.to(dev)
    d.add_(b.to(dev), alpha=2)
    d.mul_(b.to(dev))
    d.clamp_(-1, 1)
    d.t().sub_(1.0)                                                        # in-place through a view
    r = a.clone()
    r.add_(b, alpha=2).mul_(b).clamp_(-1, 1)
    r.t().sub_(1.0)
    assert torch.allclose(d.cpu(), r, atol=1e-6)
    out = torch.empty(0, device=dev)
    torch.maximum(a.to(dev), b.to(dev), out=out)
    assert torch.equal(out.cpu(), torch.maximum(a, b))
    m = torch.empty(4, 6, dtype=torch.bool, device=dev)
    torch.lt(a.to(dev), 0.0, out=m)
    assert torch.equal(m.cpu(), a < 0)
    z = torch.zeros(3, 5, dtype=torch.int64, device=dev)
    z[:, ::2].fill_(4)                                                     # strided fill
    assert z.cpu().tolist() == [[4, 0, 4, 0, 4]] * 3
    assert not bw.fallback_counts(), bw.fallback_counts()


def test_large_and_empty(bw, dev):
    a = torch.randn(3, 1 << 20)
    _check(torch.add, (a, torch.randn(3, 1)), dev)
    _check(torch.add, (torch.randn(0, 5), torch.randn(5)), dev)
    _check(torch.exp, (torch.randn(()),), dev)
