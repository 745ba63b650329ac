"""Porovik on the device: every new mechanism alone against the plain implementation's function for it, then tiny
models that differ in every size replayed whole / with a decoded tail / in portions down to two tokens / mixed on a
pool that only holds the most demanding step, the trace runner as a process, and greedy generation through ``LLM``."""
import json
import math
import os
import random

import numpy as np
import pytest
import torch

import helpers as H
import plain_porovik as P
import porovik_cases as C
from test_sobivik_gpu import DT, F64, LENS, PLAN, Bench, close, dev, env, i32, rms_err, rows_for, run_cut, weights_for

pytestmark = pytest.mark.gpu


# ---------------------------------------------------------------- the embedding

@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("hashing, width", [((101, 7, 13), 64), ((257, 1000003, 65537), 72), ((50, 3, 0), 40), (None, 48)])
def test_embedding_bigram(dtype, hashing, width):
    """Token row + hashed bigram row + position row: requests whose portions are cut anywhere (the token before a
    portion comes from the request's state slot), first tokens (the table's last row), a slot another request used
    before, multipliers whose products pass 2^31."""
    from dinfer_b200.kernels import ops
    g = torch.Generator().manual_seed(width)
    vocab, maxpos, slots = 600, 90, 3
    mk = lambda *s: (torch.randn(*s, generator=g) * 0.5).to(DT[dtype])
    table, pos = mk(vocab, width), mk(maxpos, width)
    bigram = mk(hashing[0] + 1, width) if hashing else None
    cfg = {"embedding": {"bigram": dict(zip(("buckets", "mul_prev", "mul_cur"), hashing))} if hashing else {}}
    W = {"embed": table.float(), "pos": pos.float()}
    if hashing:
        W["bigram"] = bigram.float()
    rng = random.Random(1)
    reqs = {r: [rng.randrange(vocab) for _ in range(n)] for r, n in (("a", 31), ("b", 1), ("c", 17), ("d", 40), ("e", 2))}
    want = {r: P.embed(ids, W, cfg, {"before": None, "pos": 0}) for r, ids in reqs.items()}
    plan = [{"a": 5, "b": 1}, {"a": 1, "c": 2}, {"c": 15, "a": 2, "d": 1}, {"d": 39, "a": 23}, {"e": 1}, {"e": 1}]
    slot_of, free, at = {}, list(range(slots)), {r: 0 for r in reqs}
    last = torch.full((slots + 1,), -7, dtype=torch.int32, device="cuda")
    got = {r: [] for r in reqs}
    for step in plan:
        ids, positions, cu, sl, fresh = [], [], [0], [], []
        for r, n in step.items():
            fresh.append(0 if r in slot_of else 1)
            if r not in slot_of:
                slot_of[r] = free.pop(0)
            ids += reqs[r][at[r]:at[r] + n]
            positions += list(range(at[r], at[r] + n))
            cu.append(cu[-1] + n)
            sl.append(slot_of[r])
        out = torch.empty(len(ids), width, dtype=torch.float32, device="cuda")
        ops.embedding_bigram(i32(ids), dev(table), out, dev(bigram) if hashing else None, hashing, dev(pos), i32(positions),
                             i32(cu), i32(sl), i32(fresh), last if hashing else None)
        o = 0
        for r, n in step.items():
            got[r].append(out[o:o + n].double().cpu())
            o += n
            at[r] += n
            if at[r] == len(reqs[r]):
                free.append(slot_of.pop(r))
    for r in reqs:
        assert torch.allclose(torch.cat(got[r]), want[r], atol=1e-6, rtol=1e-6), r


# ---------------------------------------------------------------- the join with norms that have a weight per coordinate

@pytest.mark.parametrize("a_dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("h", [72, 70, 256, 1000])
def test_weight_norm_join(a_dtype, h):
    """x + norm_b(a) and the next sublayer's input norm in one kernel, the norms' weights vectors stored around zero;
    widths that take the vector kernel and the scalar one; in place."""
    from dinfer_b200.kernels import stream_ops
    g = torch.Generator().manual_seed(h)
    T, eps = 6, 3e-6
    a = torch.randn(T, h, generator=g).to(DT[a_dtype])
    x = torch.randn(T, h, generator=g)
    wb, wn = torch.randn(h, generator=g) * 0.3, torch.randn(h, generator=g) * 0.3
    x_new = x.double() + P.weight_norm(a.double(), wb, eps)
    for nxt in (True, False):
        x_dev = dev(x)
        out = torch.empty(T, h, dtype=torch.bfloat16, device="cuda") if nxt else None
        stream_ops.gain_norm_join(dev(a), dev(1.0 + wb), eps, x_dev, x_dev, next_gain=dev(1.0 + wn) if nxt else None, next_out=out)
        assert torch.allclose(x_dev.double().cpu(), x_new, atol=1e-5, rtol=1e-5)
        if nxt:
            assert torch.allclose(out.double().cpu(), P.weight_norm(x_new, wn, eps), atol=3e-2, rtol=2e-2)


def test_norm_with_offset_keeps_the_stored_digits():
    """A weight stored around zero in bfloat16 is added to one in 32-bit, not rounded back."""
    import dinfer_b200.models.decoder  # noqa: F401
    from dinfer_b200.parts.base import NORMS
    n = NORMS.get("rmsnorm")({"size": 8, "eps": 1e-6, "weight": "w", "offset": 1.0}, env(8, torch.bfloat16), "")
    w = torch.tensor([0.00390625 * 1.5] * 8, dtype=torch.bfloat16, device="cuda")
    n.bind({"w": w})
    assert n.weight.dtype == torch.float32 and float(n.weight[0]) == 1.0 + 0.00390625 * 1.5


# ---------------------------------------------------------------- the recurrent mixers through their parts

SIZES = [(2, 16, 24, 64), (3, 128, 40, 96), (1, 12, 20, 72), (6, 64, 64, 128), (5, 33, 7, 40), (2, 256, 96, 64), (4, 30, 130, 64)]


def shaped(W, dtype):
    """Forget gates and decays towards one in every other channel, lower bounds inside (0, 1)."""
    for n, t in W.items():
        if n.endswith("lower"):
            t = torch.sigmoid(t * 25.0) * 0.9 + 0.05
        elif n.endswith("f.b"):
            t = t * 10.0 + torch.where(torch.arange(t.numel()) % 2 == 0, 4.0, 0.0)
        elif n.endswith("w0"):
            t = t * 10.0 - torch.where(torch.arange(t.numel()) % 2 == 0, 5.0, 0.0)
        elif n.endswith(("w2", "a.b")):
            t = t * 8.0
        W[n] = t.to(torch.bfloat16).float()
    return W


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H_, dk, dv, width", SIZES)
def test_gate_write(dtype, H_, dk, dv, width):
    """The part against the recurrence written out token by token: batches of unequal requests, portions of one and
    two tokens and of more than a staged tile, state rows that another request held before."""
    import dinfer_b200.models.decoder  # noqa: F401
    from dinfer_b200.parts.base import MIXERS
    p = {"num_heads": H_, "key_dim": dk, "value_dim": dv, "eps": 1e-5}
    names = dict(q_proj="mix.q", f_proj="mix.f", f_bias="mix.f.b", lower="mix.lower", v_proj="mix.v", norm="mix.norm", o_proj="mix.o")
    W = shaped(weights_for(MIXERS.get("gate_write")(dict(p, **names), env(width, torch.float32), "").declare(), dtype, dk, std=0.15), dtype)
    bench = Bench("gate_write", dict(p, **names), W, dtype, width, slots=4)
    inputs = rows_for(width, dtype, 11)
    got = run_cut(bench, inputs, PLAN)
    m = {"heads": H_, "dim": dk, "vdim": dv}
    for r, x in inputs.items():
        want = P.gate_write(x.double(), W, m, {"S": torch.zeros(H_, dk, dv, dtype=F64)}, 1e-5)
        close(got[r], want, dtype, r)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H_, dk, dv, width", SIZES)
def test_general_delta(dtype, H_, dk, dv, width):
    import dinfer_b200.models.decoder  # noqa: F401
    from dinfer_b200.parts.base import MIXERS
    p = {"num_heads": H_, "key_dim": dk, "value_dim": dv, "eps": 1e-5, "decay_rank": 5}
    names = dict(r_proj="mix.r", k_proj="mix.k", v_proj="mix.v", a_proj="mix.a", a_bias="mix.a.b", decay_proj=("mix.w1", "mix.w2"),
                 decay_bias="mix.w0", gate_proj="mix.g", norm="mix.norm", o_proj="mix.o")
    W = shaped(weights_for(MIXERS.get("general_delta")(dict(p, **names), env(width, torch.float32), "").declare(), dtype, dk, std=0.15), dtype)
    bench = Bench("general_delta", dict(p, **names), W, dtype, width, slots=4)
    # (rows among which no token's r lies across its k: there o = S^T r is a sum that cancels to a thousandth of its
    # terms, and the norm behind it hands the 32-bit sums' last digits on at full size, in any order of summing)
    inputs = rows_for(width, dtype, 14)
    got = run_cut(bench, inputs, PLAN)
    m = {"heads": H_, "dim": dk, "vdim": dv}
    for r, x in inputs.items():
        want = P.general_delta(x.double(), W, m, {"S": torch.zeros(H_, dk, dv, dtype=F64)}, 1e-5)
        close(got[r], want, dtype, r)


@pytest.mark.parametrize("remove", [False, True])
@pytest.mark.parametrize("widen", [1, 2])
@pytest.mark.parametrize("H_, dk, dv", [(2, 16, 24), (1, 12, 20), (3, 64, 64), (5, 33, 7), (2, 128, 40), (1, 256, 8), (1, 300, 12)])
def test_recurrence_forms(H_, dk, dv, widen, remove):
    """The kernel alone, both ways of sharing a column between lanes, against the recurrence in 64-bit: inputs that
    are views of wider rows at offsets no 16-byte load can take, requests of 1, 2, 16, 17 and 45 tokens in one batch,
    a state an earlier step left, nothing written beside the own rows."""
    from dinfer_b200.kernels import state_ops
    g = torch.Generator().manual_seed(dk * 7 + dv)
    lens = [1, 2, 16, 17, 45]
    T = sum(lens)
    n = H_ * dk
    wide = torch.randn(T, 5 * n + 3, generator=g)
    r, k = wide[:, 1:1 + n], wide[:, 1 + n:1 + 2 * n]
    w = torch.sigmoid(wide[:, 1 + 2 * n:1 + 3 * n] * 3 + 2)
    u = k.reshape(T, H_, dk)
    u = (u / u.norm(dim=-1, keepdim=True)).reshape(T, n)
    p = torch.sigmoid(wide[:, 1 + 3 * n:1 + 4 * n]) * u
    v = torch.randn(T, H_ * dv + 1, generator=g)[:, 1:]
    S0 = torch.randn(len(lens), H_, dk, dv, generator=g) * 0.3
    state = torch.full((len(lens) + 2, n * dv + 3), float("nan"), device="cuda")
    slots = [4, 0, 2, 5, 1]
    fresh = [1, 0, 0, 1, 0]
    for b, s in enumerate(slots):
        if not fresh[b]:
            state[s, :n * dv] = dev(S0[b].reshape(-1))
    stack = dev(torch.cat([r, k, w, u, p], dim=1))           # views at column offsets that are no multiple of 4 when n is not
    cols = [stack[:, i * n:(i + 1) * n] for i in range(5)]
    vd = dev(v)
    cu = [0]
    for x in lens:
        cu.append(cu[-1] + x)
    kw = dict(k=cols[1], u=cols[3], p=cols[4]) if remove else {}
    out = state_ops.recurrence(cols[0], cols[2], vd, state, i32(cu), i32(slots), i32(fresh), H_, dk, dv, widen=widen, **kw).double().cpu()
    for b, (lo, hi) in enumerate(zip(cu, cu[1:])):
        S = torch.zeros(H_, dk, dv, dtype=F64) if fresh[b] else S0[b].double()
        for t in range(lo, hi):
            rr, kk, ww, uu, pp = (x[t].double().reshape(H_, dk) for x in (r, k, w, u, p))
            vv = v[t].double().reshape(H_, dv)
            if remove:
                seen = torch.einsum("hkv,hk->hv", S, uu)
                S = ww[:, :, None] * S - pp[:, :, None] * seen[:, None, :] + kk[:, :, None] * vv[:, None, :]
            else:
                S = ww[:, :, None] * S + (1 - ww)[:, :, None] * vv[:, None, :]
            assert torch.allclose(out[t], torch.einsum("hkv,hk->hv", S, rr), atol=2e-5, rtol=2e-5), (b, t)
        assert torch.allclose(state[slots[b], :n * dv].double().cpu(), S.reshape(-1), atol=2e-5, rtol=2e-5)
        assert torch.isnan(state[slots[b], n * dv:]).all()
    assert torch.isnan(state[3]).all() and torch.isnan(state[6]).all()


@pytest.mark.parametrize("remove", [False, True])
def test_recurrence_remembers_a_far_token(remove):
    """A value written at the first token is read back 300 tokens later, through portions and decoded tokens, with a
    query that only the first key's channel answers: a channel that hardly decays (the delta rule), or one whose gate
    stays shut after the first token (gate-write: an open gate would also write)."""
    from dinfer_b200.kernels import state_ops
    T, dk, dv = 301, 16, 8
    g = torch.Generator().manual_seed(1)
    v = torch.randn(T, dv, generator=g)
    r, k, w = torch.zeros(T, dk), torch.zeros(T, dk), torch.full((T, dk), 0.5)
    w[:, 3] = 0.999
    if remove:
        k[0, 3] = 1.0
        k[1:, 5] = 1.0                                       # every later key lies across the first
    else:
        w[0, 3] = 0.0                                        # gate-write: what is written is 1 - f
        w[1:, 3] = 1.0
    r[T - 1, 3] = 1.0
    u, p = k.clone(), 0.9 * k
    state = torch.full((3, dk * dv + 5), float("nan"), device="cuda")
    at, outs = 0, []
    for n in (1, 2, 40, 33, 1, 1, 200, 22, 1):
        sl = slice(at, at + n)
        kw = dict(k=dev(k[sl]), u=dev(u[sl]), p=dev(p[sl])) if remove else {}
        o = state_ops.recurrence(dev(r[sl]), dev(w[sl]), dev(v[sl]), state, i32([0, n]), i32([1]), i32([1 if at == 0 else 0]),
                                 1, dk, dv, **kw)
        outs.append(o.cpu())
        at += n
    got = torch.cat(outs)[T - 1, 0]
    assert torch.allclose(got, v[0] * (0.999 ** 300 if remove else 1.0), atol=1e-6, rtol=1e-4)
    assert torch.isnan(state[1, dk * dv:]).all() and torch.isnan(state[0]).all()


# ---------------------------------------------------------------- attention with a distance bias, a temperature and a gate

ATT = [  # heads, kv heads, dim, vdim, temperature, page size
    (4, 2, 8, 16, (0.7, 5), 16), (6, 1, 24, 40, (0.3, 1), 4), (3, 3, 10, 6, None, 16), (4, 1, 64, 64, (0.5, 16), 16),
    (2, 2, 32, 32, None, 8), (4, 2, 128, 128, (0.6, 48), 16), (1, 1, 40, 24, (0.4, 7), 64)]


def att_params(H_, G, D, V, temp):
    p = {"num_heads": H_, "num_kv_heads": G, "head_dim": D, "v_dim": V, "scale": 0.8 * D ** -0.5, "distance_slopes": "geometric",
         "gate_proj": "mix.g", "q_proj": "mix.q", "k_proj": "mix.k", "v_proj": "mix.v", "o_proj": "mix.o"}
    if temp:
        p["q_temperature"] = temp
    return p


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H_, G, D, V, temp, block_size", ATT)
def test_biased_attention(dtype, H_, G, D, V, temp, block_size):
    """The attention part with the design's options against the plain formula: grouped heads, keys and values of
    different widths (plain-arithmetic kernel) and of one width (tensor-core kernel in bfloat16), prompts beside
    portions behind a history beside decoded tokens."""
    import dinfer_b200.models.decoder  # noqa: F401
    from dinfer_b200.parts.base import MIXERS
    width = 64
    p = att_params(H_, G, D, V, temp)
    W = weights_for(MIXERS.get("gqa_attention")(p, env(width, torch.float32), "").declare(), dtype, D + V, std=0.12,
                    scale={"mix.q": 5.0})
    bench = Bench("gqa_attention", p, W, dtype, width, block_size=block_size, num_blocks=4096 // block_size)
    bench.binding.kv.zero_()         # as the engine makes it: the TMA kernels fetch whole pages, and 0 * NaN is no 0
    inputs = rows_for(width, dtype, 5)
    got = run_cut(bench, inputs, PLAN)
    m = {"heads": H_, "kv_heads": G, "dim": D, "vdim": V, "scale": p["scale"]}
    if temp:
        m["q_temp"] = {"coef": temp[0], "every": temp[1]}
    for r, x in inputs.items():
        want, _ = P.biased_attention(x.double(), W, m, {"k": torch.zeros(0, G, D, dtype=F64), "v": torch.zeros(0, G, V, dtype=F64)})
        close(got[r], want, dtype, r)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("D", [24, 64])
@pytest.mark.parametrize("far", [0, 15, 16, 17, 63, 64])
def test_attention_finds_a_far_key(dtype, D, far):
    """One key far back (at and around page borders) answers the query more strongly than the distance bias takes off:
    the output is that token's value, from a prompt's last row and from a decoded token alike.  Identity projections
    make the rows themselves the queries, keys and values."""
    width = D
    eye = torch.eye(D)
    p = {"num_heads": 1, "num_kv_heads": 1, "head_dim": D, "v_dim": D, "scale": 1.0, "distance_slopes": "geometric",
         "gate_proj": "mix.g", "q_proj": "mix.q", "k_proj": "mix.k", "v_proj": "mix.v", "o_proj": "mix.o"}
    W = {"mix.q": eye * 8.0, "mix.k": eye, "mix.v": eye, "mix.g": torch.zeros(D, D), "mix.o": eye}
    T = 330
    g = torch.Generator().manual_seed(D + far)
    x = torch.zeros(T, D)
    x[:, 1:] = torch.randn(T, D - 1, generator=g) * 0.05     # every row's first element is zero but the far one's
    x[far, 0] = 4.0
    x[far, 1:] = torch.randn(D - 1, generator=g)
    x[T - 2:, 0] = 1.0                                       # the asking rows: score 8 * 4 = 32 at the far key, bias about 1.3
    x = x.to(DT[dtype]).float()
    for tail in (0, 1):                                      # the asking row as a prompt's last row, or decoded alone
        bench = Bench("gqa_attention", p, W, dtype, width, block_size=16, num_blocks=64)
        bench.binding.kv.zero_()
        if tail:
            bench.run([("a", x[:T - 1])])
            out = bench.run([("a", x[T - 1:])])[-1]
        else:
            out = bench.run([("a", x)])[-1]
        want, _ = P.biased_attention(x.double(), W, {"heads": 1, "dim": D, "scale": 1.0},
                                     {"k": torch.zeros(0, 1, D, dtype=F64), "v": torch.zeros(0, 1, D, dtype=F64)})
        close(out, want[-1], dtype)
        assert float((out[1:] * 2 - x[far, 1:].double()).abs().max()) < 0.15   # half (the gate) of the far token's row


# ---------------------------------------------------------------- experts whose weight multiplies the input

@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("E, top, ff, width, T", [(4, 2, 24, 64, 37), (3, 1, 16, 72, 5), (5, 5, 12, 40, 64), (8, 2, 64, 128, 1)])
def test_experts_weighted_on_the_input(dtype, E, top, ff, width, T):
    import dinfer_b200.models.decoder  # noqa: F401
    from dinfer_b200.parts.base import FEED_FORWARDS
    p = {"num_experts": E, "top_k": top, "expert_size": ff, "activation": "silu", "gated": True, "scoring": "sigmoid",
         "renormalize": False, "weight_on": "input", "router": "mlp.router", "expert_gate": "mlp.e{e}.gate",
         "expert_up": "mlp.e{e}.up", "expert_down": "mlp.e{e}.down"}
    part = FEED_FORWARDS.get("moe")(p, env(width, DT[dtype]), "")
    W = weights_for(part.declare(), dtype, E + top, std=0.2, scale={"mlp.router": 4.0})
    part.bind({k: dev(v, DT[dtype]) for k, v in W.items()})
    x = (torch.randn(T, width, generator=torch.Generator().manual_seed(T)) * 1.5).to(DT[dtype]).float()
    got = part.forward(dev(x, DT[dtype])).double().cpu()
    want = P.expert_ff(x.double(), W, {"router": {"experts": E, "top": top}})
    close(got, want, dtype)
    if T < 5:
        return
    # the weight on the output would give something else
    other = FEED_FORWARDS.get("moe")(dict(p, weight_on="output"), env(width, DT[dtype]), "")
    other.bind({k: dev(v, DT[dtype]) for k, v in W.items()})
    assert float((other.forward(dev(x, DT[dtype])).double().cpu() - want).abs().max()) > 0.02 * float(want.abs().max())


# ---------------------------------------------------------------- whole models

LENGTHS = {"A": {"a": 1, "b": 2, "c": 45, "d": 131, "e": 77},
           "B": {"a": 150, "b": 3, "c": 66, "d": 1, "e": 19},
           "C": {"a": 97, "b": 40, "c": 2, "d": 71},
           "D": {"a": 120, "b": 1, "c": 33, "d": 64},
           "E": {"a": 190, "b": 17, "c": 65, "d": 128}}
BF16_WORST, BF16_RMS, BF16_OVER = 0.3, 0.1, 0.15


class Oracle:
    def __init__(self, model_dir):
        self.cfg = json.load(open(os.path.join(model_dir, "config.json")))
        self.W = C.load_weights(model_dir)
        self._cache = {}

    def logits(self, ids):
        key = tuple(ids)
        if key not in self._cache:
            self._cache[key] = P.forward(self.cfg, self.W, list(ids), P.new_state(self.cfg)).numpy()
        return self._cache[key]


@pytest.fixture(scope="module")
def model_dirs(tmp_path_factory):
    out = {}
    for name, cfg in C.CONFIGS.items():
        for dt in DT:
            out[(name, dt)] = C.write_model(str(tmp_path_factory.mktemp(f"porovik{name}_{dt}")), cfg, 11 + ord(name), DT[dt])
    return out


_REQUESTS = {}


def requests(name, model_dirs):
    if name not in _REQUESTS:
        cfg, rng = C.CONFIGS[name], random.Random(7 + ord(name))
        oracle = Oracle(model_dirs[(name, "bfloat16")])
        tokens = {r: H.random_tokens(rng, n, cfg["vocab"]) for r, n in LENGTHS[name].items()}
        _REQUESTS[name] = (tokens, {r: oracle.logits(t) for r, t in tokens.items()})
    return _REQUESTS[name]


@pytest.mark.parametrize("block_size", [4, 16, 64])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(C.CONFIGS))
def test_replay_all_ways(model_dirs, name, dtype, block_size):
    """Every position of every request: whole / with a decoded tail long enough to pass page borders / in portions
    down to two tokens / mixed with up to four live requests (some sitting steps out) on a pool that only holds the
    most demanding step, so that pages and state slots are freed and used again."""
    model_dir = model_dirs[(name, dtype)]
    rng = random.Random(99 + ord(name))
    lengths = LENGTHS[name]
    tokens, want = requests(name, model_dirs)
    schedules = {
        "whole": H.schedule_whole(lengths),
        "tail": H.schedule_tail(lengths, 70),
        "chunks": H.schedule_chunks(lengths, rng),
        "mixed": H.schedule_mixed(lengths, rng),
        "mixed2": H.schedule_mixed(dict(reversed(list(lengths.items()))), rng, max_live=3, decode_tail=40),
    }
    max_tokens = max(H.max_live_tokens(s, round_to=max(64, block_size)) for s in schedules.values())
    rp = H.LocalReplay(model_dir, dtype, max_tokens, block_size=block_size)
    worst, spread, over = {}, {}, {}
    for sname, steps in schedules.items():
        got = H.run_schedule(rp, steps, tokens, tag=sname + "/")
        worst[sname] = max(H.rel_err(got[r], want[r]) for r in tokens)
        rows = np.concatenate([np.abs(got[r].astype(np.float64) - want[r]).max(axis=1) / np.abs(want[r]).max() for r in tokens])
        keep = rows <= BF16_WORST
        over[sname] = float(1.0 - keep.mean()) if np.isfinite(rows).all() else 1.0
        g, w = np.concatenate([got[r] for r in tokens])[keep], np.concatenate([want[r] for r in tokens])[keep]
        spread[sname] = rms_err(g, w) if keep.any() else float("inf")
    assert rp.close() == 0
    # 32-bit is the sharp test.  In bfloat16 a rounding can travel far in this design (every sublayer's output is
    # normed back to unit size, its relative error included), and a router whose two best scores lie closer than a
    # rounding picks another expert for that token than the 64-bit implementation does (seen in these models: single
    # tokens whose feed-forward result jumps in a layer with experts, then fades through the states).  So there: at
    # most BF16_OVER of the positions may differ by more than BF16_WORST of the logits' largest, and over the others
    # the root mean square of the differences is held to BF16_RMS of the logits' own (a fault gives about 1 everywhere;
    # faults at single places are the 32-bit runs' and the mechanisms' own tests' to find).
    if dtype == "float32":
        bad = {k: v for k, v in worst.items() if not v <= H.TOLERANCE[dtype]}
    else:
        bad = {k: (over[k], spread[k]) for k in worst if not (over[k] <= BF16_OVER and spread[k] <= BF16_RMS)}
    assert not bad, f"{name} {dtype} pages of {block_size}: {bad} (largest: {worst}; over: {over}; rms: {spread})"


def test_residual_stream_layer_by_layer(model_dirs):
    """The 32-bit engine's residual stream after every layer against the plain implementation's, a prompt in two
    portions and a decoded token."""
    from dinfer_b200.config.engine_config import EngineConfig
    from dinfer_b200.engine.batch import StepEntry
    from dinfer_b200.engine.runner import ModelRunner
    from dinfer_b200.parts.block import SandwichResidual
    model_dir = model_dirs[("A", "float32")]
    cfg = C.CONFIGS["A"]
    ids = H.random_tokens(random.Random(3), 40, cfg["vocab"])
    want = []
    P.forward(cfg, C.load_weights(model_dir), ids, P.new_state(cfg), residuals=want)
    runner = ModelRunner.from_dir(model_dir, EngineConfig(max_model_len=64, max_num_seqs=2, max_num_batched_tokens=64, num_blocks=8,
                                                          block_size=16, dtype="float32", enable_cuda_graph=False))
    seen = []
    plain_forward = SandwichResidual.forward

    def spy(self, stream, ctx, cache, next_block=None):
        plain_forward(self, stream, ctx, cache, next_block)
        seen.append(stream.x.double().cpu().clone())
    SandwichResidual.forward = spy
    try:
        for lo, hi in ((0, 25), (25, 39), (39, 40)):
            runner.step([StepEntry("r", ids[lo:hi], [])])
    finally:
        SandwichResidual.forward = plain_forward
    L = len(cfg["layers"])
    for i in range(L):
        got = torch.cat([seen[s * L + i] for s in range(3)])
        assert torch.allclose(got, want[i], atol=2e-4, rtol=2e-4), i


def test_trace_runner_and_first_tokens(model_dirs, tmp_path):
    """Through ``bin/trace_run`` as a process: the first tokens of sequences (a request of one token, the first two
    positions of others), and a request that sits steps out while others come and go."""
    model_dir = model_dirs[("A", "float32")]
    cfg = C.CONFIGS["A"]
    rng = random.Random(5)
    tokens = {r: H.random_tokens(rng, n, cfg["vocab"]) for r, n in {"p": 1, "q": 2, "r": 70, "s": 45}.items()}
    oracle = Oracle(model_dir)
    rp = H.Replay(model_dir, "float32", str(tmp_path / "out"), 256)
    try:
        a = rp.step([{"id": "p", "tokens": tokens["p"], "want": [0]}, {"id": "r", "tokens": tokens["r"][:2], "want": [0, 1]}], ["p"])
        b = rp.step([{"id": "q", "tokens": tokens["q"], "want": [0, 1]}, {"id": "s", "tokens": tokens["s"][:40], "want": [39]}], ["q"])
        c = rp.step([{"id": "r", "tokens": tokens["r"][2:], "want": [67]}, {"id": "s", "tokens": tokens["s"][40:41], "want": [0]}], ["r"])
        d = rp.step([{"id": "s", "tokens": tokens["s"][41:], "want": [3]}], ["s"])
    finally:
        assert rp.close() == 0
    for got, want in ((a[0], oracle.logits(tokens["p"])[0]), (a[1:], oracle.logits(tokens["r"])[:2]),
                      (b[:2], oracle.logits(tokens["q"])), (b[2], oracle.logits(tokens["s"])[39]),
                      (c[0], oracle.logits(tokens["r"])[69]), (c[1], oracle.logits(tokens["s"])[40]),
                      (d[0], oracle.logits(tokens["s"])[44])):
        assert H.rel_err(np.asarray(got), np.asarray(want)) <= H.TOLERANCE["float32"]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "E"])
def test_greedy_generation_through_the_entry_point(model_dirs, name, dtype):
    """``LLM.generate``: scheduler, chunked prompts (a token budget below the prompts' lengths), decode steps replayed
    as CUDA graphs (the mixers' state and the embedding's token before are driven from device tensors), greedy
    sampling; more requests than run at once; long decoding."""
    from dinfer_b200 import LLM, SamplingParams
    model_dir = model_dirs[(name, dtype)]
    cfg = C.CONFIGS[name]
    rng = random.Random(21)
    prompts = [H.random_tokens(rng, n, cfg["vocab"]) for n in (1, 5, 23, 40, 9, 31)]
    llm = LLM(model_dir, dtype=dtype, max_model_len=160, max_num_seqs=4, max_num_batched_tokens=16, block_size=16,
              num_blocks=48)
    outs = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=80, ignore_eos=True))
    oracle = Oracle(model_dir)
    exact = total = 0
    for p, o in zip(prompts, outs):
        assert len(o.output_ids) == 80
        lg = oracle.logits(list(p) + list(o.output_ids))
        exact += sum(int(lg[len(p) - 1 + i].argmax()) == t for i, t in enumerate(o.output_ids))
        total += 80
    assert exact >= (0.8 if dtype == "bfloat16" else 0.99) * total, (exact, total)
    assert any(isinstance(k, int) for k in llm.runner._graphs)
