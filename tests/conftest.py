import os
import sys

# The tokenizer (like the reference's) asks the process locale for the class of code points outside its own tables;
# the golden vectors were made under the C locale.
os.environ["LC_ALL"] = "C"

import numpy as np  # noqa: E402
import pytest  # noqa: E402

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
import __graft_entry__ as entry  # noqa: E402


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200; run with -m gpu")


@pytest.fixture(scope="session")
def qb():
    """The product package (ctypes binding of the C ABI)."""
    return entry.load_package()


@pytest.fixture(scope="session")
def orc():
    """The CPU oracle (test infrastructure)."""
    return entry.load_oracle()


@pytest.fixture(scope="session")
def ctx(qb):
    c = qb.Context(0)
    yield c
    c.close()


@pytest.fixture(autouse=True)
def _release_device_arrays(request):
    yield
    if "ctx" in request.fixturenames:
        c = request.getfixturevalue("ctx")
        c.sync()
        c.release_arrays()


@pytest.fixture(scope="session")
def ref():
    """The reference's own CUDA kernels (oracle/_ref/libqw3ref.so), or None if not built."""
    import ctypes
    path = os.path.join(ROOT, "oracle", "_ref", "libqw3ref.so")
    if not os.path.exists(path):
        return None
    return ctypes.CDLL(path)


def std_mt19937_uniform(rs, n, a, b):
    """n draws of std::uniform_real_distribution<float>(a, b) on a std::mt19937 (libstdc++):
    one 32-bit output per value, u = float(raw) / 2^32 (clamped below 1), x = u * (b - a) + a."""
    raw = rs._bit_generator.random_raw(n).astype(np.uint32)
    u = raw.astype(np.float32) / np.float32(4294967296.0)
    u = np.minimum(u, np.nextafter(np.float32(1.0), np.float32(0.0)))
    return (u * np.float32(b - a) + np.float32(a)).astype(np.float32)


def tiny_ocfg(orc, qb):
    return orc.ModelConfig(**qb.configs.tiny().as_dict())


@pytest.fixture(scope="session")
def ref_attn():
    """The reference's native decode attention (oracle/_ref/libqw3ref_attn.so, `make -C oracle ref-attn`), or None."""
    import ctypes
    path = os.path.join(ROOT, "oracle", "_ref", "libqw3ref_attn.so")
    if not os.path.exists(path):
        return None
    return ctypes.CDLL(path)


def rel_err(got, want):
    """max |got - want| / max |want|: the relative logit error the step is specified in."""
    return float(np.abs(got - want).max() / np.abs(want).max())


def top2_margin(lg):
    top = np.sort(lg)[-2:]
    return float((top[1] - top[0]) / np.abs(lg).max())


def noise_cap(floor, tol=1e-2, slack=1.5):
    """Bound for a max-relative logit error given the measured one-ulp noise floor of the model: the specified
    tolerance, or `slack` x the largest floor sample where the model's own rounding noise is above it (the floor is a
    maximum over a few steps of a heavy-tailed quantity; an error in the wiring moves logits by tens of percent)."""
    return max(tol, slack * max(floor))


def greedy_noise_floor(orc, omodel, prompt, steps, chunk=0, max_ctx=None):
    """Noise floor of a model under the smallest change an equally valid fp32 implementation could make: the logits of
    `steps` teacher-forced greedy steps with every attn_norm gain of layer 0 moved by one unit in the last place,
    against the unmoved model.  Returns the per-step max-relative logit differences.  The network re-quantises its
    activations to int8 before every projection, so the move flips rounding decisions and the difference is the
    rounding noise itself."""
    max_ctx = max_ctx or len(prompt) + steps + 8
    a = orc.Seq(omodel, max_ctx)
    a.prefill(prompt, chunk)
    base, toks = [a.last_logits(1)[0].copy()], [a.cur_token]
    for _ in range(steps - 1):
        a.greedy_step()
        base.append(a.last_logits(1)[0].copy())
        toks.append(a.cur_token)
    omodel.nudge_attn_norm(0, 1)
    try:
        b = orc.Seq(omodel, max_ctx)
        b.prefill(prompt, chunk)
        errs = []
        for i in range(steps):
            if i:
                b.greedy_step()
            errs.append(rel_err(b.last_logits(1)[0], base[i]))
            b.set_cur_token(toks[i])
    finally:
        omodel.nudge_attn_norm(0, -1)
    return errs
