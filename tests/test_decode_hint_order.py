"""Host logic of the decode step's next-weights hints (no GPU): before every call the step must name exactly the
weights of the call AFTER it, the last call of a step names the first call of the next step, and a step with more
than one activation row, or with hints switched off, names nothing."""
import pytest

torch = pytest.importorskip("torch")

from boostr_b200 import decode_stack as ds  # noqa: E402


class _W:
    def __init__(self, name):
        self.name = name


class _Lin:
    def __init__(self, name, log):
        self.weight, self._log = _W(name), log

    def forward(self, x, out=None):
        self._log.append(("call", (self.weight.name,)))
        return out

    def forward_gathered(self, x, out, exchange, local=None):
        self._log.append(("call", (self.weight.name,)))
        return out


def _fake_stack(log, m, layers, world=1):
    st = object.__new__(ds.DecodeStack)
    st.m, st.world, st.prefetch, st.exchange = m, world, True, None
    st.layers = []
    for i in range(layers):
        L = {n: _Lin(f"{n}{i}", log) for n in ("q", "k", "v", "o", "gate", "up", "down")}
        L["qkv"] = [L["q"], L["k"], L["v"]]
        st.layers.append(L)
    st.lm_head = _Lin("lm_head", log)
    for n in ("x", "q", "k", "v", "o", "h", "d", "logits", "logits_local"):
        setattr(st, n, None)
    return st


@pytest.fixture
def patched(monkeypatch):
    log = []
    monkeypatch.setattr(ds.ops, "prefetch_next", lambda ws, swiglu=False: log.append(("hint", tuple(w.name for w in ws), swiglu)))
    monkeypatch.setattr(ds.ops, "quant_swiglu", lambda x, g, u, out=None: log.append(("call", (g.name, u.name))) or out)
    monkeypatch.setattr(ds.QuantLinear, "forward_batch",
                        staticmethod(lambda ls, x, outs=None: log.append(("call", tuple(l.weight.name for l in ls))) or outs))
    return log


@pytest.mark.parametrize("world", [1, 2])
def test_every_call_is_told_what_follows_it(patched, world):
    st = _fake_stack(patched, 1, 3, world)
    st.step()
    calls = [e for e in patched if e[0] == "call"]
    hints = [e for e in patched if e[0] == "hint"]
    assert len(calls) == len(hints) == 3 * 4 + 1
    # strictly alternating, the hint first
    assert [e[0] for e in patched] == ["hint", "call"] * len(calls)
    for i, h in enumerate(hints):
        nxt = calls[(i + 1) % len(calls)]  # the last call of the step is followed by the first call of the next step
        assert h[1] == nxt[1], (i, h, nxt)
        assert h[2] == (len(nxt[1]) == 2), "only the gate/up pair is a SwiGLU hint"


def test_no_hints_for_several_rows_or_when_switched_off(patched):
    st = _fake_stack(patched, 4, 2)
    st.step()
    assert all(e[0] == "call" for e in patched) and len(patched) == 9
    del patched[:]
    st = _fake_stack(patched, 1, 2)
    st.prefetch = False
    st.step()
    assert all(e[0] == "call" for e in patched) and len(patched) == 9
