"""Bokenex on the GPU against the plain float64 restatement in ``oracle/bokenex.py`` (no code shared with the package).

Kernel level: every mechanism alone, with inputs built so that a fault shows (one key that dominates the output placed
just inside / just outside a window, at a page border, far back; state carried over portions of 1, 2, 3 tokens).
Engine level, through ``CausalLMEngine`` and its scheduler: whole prompts, token-by-token decoding, portions, mixed
batches, reuse of pages and state slots, long decoding across pages and windows, odd sizes, greedy generation, CUDA
graphs against eager.  The float32 engine is the sharp comparison; bfloat16 is checked against its rounding noise."""
import math

import pytest
import torch

from oracle import bokenex as O

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
F64 = torch.float64


@pytest.fixture(scope="module")
def nat():
    import nano_qwen3tts_vllm_b200._native as n
    n.lib()
    return n


class Lay:
    """A hand-made step layout for kernel tests: sequences [(pos0, n_new, slot, block_table)]."""

    def __init__(self, seqs, page, max_blocks):
        tok_seq, pos, slots, start = [], [], [], []
        o = 0
        for b, (p0, n, _, bt) in enumerate(seqs):
            start.append(o)
            for t in range(n):
                p = p0 + t
                tok_seq.append(b), pos.append(p), slots.append(bt[p // page] * page + p % page)
            o += n
        i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
        self.tok_seq, self.positions, self.slot_mapping = i32(tok_seq), i32(pos), i32(slots)
        self.seq_start, self.seq_pos0 = i32(start), i32([s[0] for s in seqs])
        self.seq_len, self.seq_slot = i32([s[1] for s in seqs]), i32([s[2] for s in seqs])
        bt = torch.zeros(len(seqs), max_blocks, dtype=torch.int32)
        for b, s in enumerate(seqs):
            bt[b, :len(s[3])] = torch.tensor(s[3], dtype=torch.int32)
        self.block_tables = bt.to(DEV)
        self.n_tokens, self.n_seqs, self.max_new = o, len(seqs), max(s[1] for s in seqs)


def rel(a, b):
    return ((a.double().cpu() - b.double().cpu()).abs().max() / b.double().abs().max().clamp_min(1e-30)).item()


# ------------------------------------------------------------------------------------------------ mechanisms alone
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("cols", [40, 256, 1000])
def test_embed_residual_and_gain_norm(nat, dtype, cols):
    g = torch.Generator().manual_seed(cols)
    n, vocab, maxpos, top = 7, 19, 23, 3
    emb = torch.randn(vocab, cols, generator=g).to(dtype)
    pos = torch.randn(maxpos, cols, generator=g).to(dtype)
    tok = torch.randint(0, vocab, (n,), generator=g).int()
    p = torch.randint(0, maxpos, (n,), generator=g).int()
    gain = torch.tensor([1.37])
    eps = 1e-3
    x = torch.empty(n, cols, device=DEV)
    h = torch.empty(n, cols, dtype=dtype, device=DEV)
    nat.embed_pos_norm(tok.to(DEV), p.to(DEV), emb.to(DEV), pos.to(DEV), x, h, gain.to(DEV), eps)
    x_ref = emb.double()[tok.long()] + pos.double()[p.long()]
    assert rel(x, x_ref) < 1e-6
    tol = 1e-5 if dtype == torch.float32 else 1e-2
    assert rel(h, O.gain_rms_norm(x_ref, gain.double(), eps)) < tol
    # residual update with every optional term, then the next norm
    a = torch.randn(n, cols, generator=g).to(dtype)
    b = torch.randn(n, cols, generator=g).to(dtype)
    z = torch.randn(n * top, cols, generator=g).to(dtype)
    zw = torch.rand(n, top, generator=g)
    for use in [(1, 1, 1), (1, 0, 0), (1, 1, 0), (1, 0, 1), (0, 0, 0)]:
        xx = x_ref.float().to(DEV)
        hh = torch.empty(n, cols, dtype=dtype, device=DEV)
        nat.residual_norm(xx, a.to(DEV) if use[0] else None, b.to(DEV) if use[1] else None, z.to(DEV) if use[2] else None,
                          zw.to(DEV) if use[2] else None, 0.7, hh, gain.to(DEV), eps, dtype)
        s = use[0] * a.double() + use[1] * b.double() + use[2] * (zw.double()[:, :, None] * z.double().view(n, top, cols)).sum(1)
        ref = x_ref.float().double() + 0.7 * s
        assert rel(xx, ref) < 1e-5
        assert rel(hh, O.gain_rms_norm(ref, gain.double(), eps)) < tol
    rows = torch.tensor([4, 0, 4], dtype=torch.int32)
    out = nat.gather_gain_norm(x, rows.to(DEV), gain.to(DEV), eps, dtype)
    assert rel(out, O.gain_rms_norm(x_ref[rows.long()], gain.double(), eps)) < tol
    y = torch.randn(5, 33, generator=g).to(dtype)
    assert rel(nat.relu_sq_(y.clone().to(DEV)), O.relu_squared(y.double()).to(dtype)) < 1e-6


@pytest.mark.parametrize("taps", [1, 2, 4, 5])
@pytest.mark.parametrize("H,G,d,dv", [(4, 2, 24, 40), (3, 3, 32, 8), (8, 1, 64, 64)])
def test_short_conv_head_norm_cache_write_in_portions(nat, taps, H, G, d, dv):
    """The convolution over a sequence cut into portions (1, 2, 3, 7 ... tokens) with its carried state, in a state
    slot that another sequence used before, beside a second sequence; k and v land in scattered pages."""
    g = torch.Generator().manual_seed(taps * 100 + d)
    page, T, eps = 16, 45, 1e-4
    C = H * d + G * d + G * dv
    u = [torch.randn(T, C, generator=g), torch.randn(T, C, generator=g)]
    w = torch.randn(C, taps, generator=g)
    qn, kn = torch.rand(d, generator=g) + 0.5, torch.rand(d, generator=g) + 0.5
    tables = [[5, 2, 7], [0, 6, 3]]
    state = torch.full((3, max(taps - 1, 1), C), 7.0, device=DEV)            # garbage of an earlier owner
    kc = torch.zeros(8, page, G * d, device=DEV)
    vc = torch.zeros(8, page, G * dv, device=DEV)
    cuts = [1, 2, 3, 7, 1, 1, 12, 2, 16]
    got_q = [[], []]
    at = 0
    for n in cuts:
        lay = Lay([(at, n, 2, tables[0]), (at, n, 0, tables[1])], page, 3)
        uu = torch.cat([u[0][at:at + n], u[1][at:at + n]]).to(DEV)
        q = torch.empty(2 * n, H * d, device=DEV)
        nat.conv_headnorm_kvwrite(uu, w.to(DEV), state, lay, qn.to(DEV), kn.to(DEV), q, kc, vc, H, G, d, dv, taps, eps)
        got_q[0].append(q[:n].cpu()), got_q[1].append(q[n:].cpu())
        at += n
    assert at == T
    for s in range(2):
        y = O.causal_short_conv(u[s].double(), w.double())
        q_ref = O.vector_rms_norm(y[:, :H * d].view(T, H, d), qn.double(), eps).reshape(T, -1)
        k_ref = O.vector_rms_norm(y[:, H * d:H * d + G * d].view(T, G, d), kn.double(), eps).reshape(T, -1)
        v_ref = y[:, H * d + G * d:]
        assert rel(torch.cat(got_q[s]), q_ref) < 1e-5
        slots = torch.tensor([tables[s][p // page] * page + p % page for p in range(T)])
        assert rel(kc.view(-1, G * d)[slots], k_ref) < 1e-5
        assert rel(vc.view(-1, G * dv)[slots], v_ref) < 1e-5


def _attn_case(nat, H, G, d, dv, window, page, seqs, dtype=torch.float32, spike=None, seed=0):
    """seqs: [(cached tokens, new tokens)].  Fills the cache with the sequences' keys, runs the kernel for the new
    tokens, compares with the plain implementation over the whole sequence.  ``spike`` = (sequence, key position):
    that key gets a huge value vector and a score that saturates the sigmoid for every query."""
    g = torch.Generator().manual_seed(seed)
    nb = [math.ceil((c + n) / page) for c, n in seqs]
    perm = torch.randperm(sum(nb) + 3, generator=g).tolist()
    tables, o = [], 0
    for k in nb:
        tables.append(perm[o:o + k])
        o += k
    kc = torch.zeros(sum(nb) + 3, page, G * d, dtype=dtype, device=DEV)
    vc = torch.zeros(sum(nb) + 3, page, G * dv, dtype=dtype, device=DEV)
    r1 = (torch.rand(H, generator=g) * 0.8).float()
    r2 = (torch.rand(H, generator=g) + 0.1).float()
    pb = (torch.randn(H, generator=g) - 1.0).float()
    scale = 0.37
    qs, refs = [], []
    for s, (c, n) in enumerate(seqs):
        T = c + n
        q = torch.randn(T, H, d, generator=g).to(dtype)
        k = torch.randn(T, G, d, generator=g).to(dtype)
        v = torch.randn(T, G, dv, generator=g).to(dtype)
        if spike is not None and spike[0] == s:
            j = spike[1]
            k[j] = 0
            k[j, :, 0] = 64.0
            q[:, :, 0] = 4.0                      # score 4 * 64 * scale: weight 1 whatever the distance bias
            v[j] = 1000.0
        slots = torch.tensor([tables[s][p // page] * page + p % page for p in range(T)], device=DEV)
        kc.view(-1, G * d)[slots] = k.view(T, -1).to(DEV)
        vc.view(-1, G * dv)[slots] = v.view(T, -1).to(DEV)
        qs.append(q[c:].reshape(n, -1))
        refs.append(O.windowed_sigmoid_attention(q.double(), k.double(), v.double(), scale, window, r1.double(), r2.double(),
                                                 pb.double())[c:].reshape(n, -1))
    lay = Lay([(c, n, 0, tables[s]) for s, (c, n) in enumerate(seqs)], page, max(nb))
    qd = torch.cat(qs).to(DEV)
    out = torch.empty(qd.shape[0], H * dv, dtype=dtype, device=DEV)
    nat.window_sigmoid_attn(qd, kc, vc, out, lay, r1.to(DEV), r2.to(DEV), pb.to(DEV), H, G, d, dv, page, window, scale)
    return out, torch.cat(refs)


@pytest.mark.parametrize("H,G,d,dv", [(8, 1, 64, 64), (4, 2, 24, 40), (3, 3, 130, 200), (8, 2, 16, 12)])
@pytest.mark.parametrize("window", [1, 5, 33, 100])
def test_window_sigmoid_attention_mixed_batch(nat, H, G, d, dv, window):
    out, ref = _attn_case(nat, H, G, d, dv, window, 16, [(0, 50), (37, 1), (20, 23), (63, 2), (0, 1)], seed=window)
    assert rel(out, ref) < 2e-5
    out, ref = _attn_case(nat, H, G, d, dv, window, 16, [(0, 50), (37, 1)], dtype=torch.bfloat16, seed=window)
    assert rel(out, ref) < 2e-2


@pytest.mark.parametrize("window,page", [(9, 8), (16, 16), (17, 16), (40, 16), (64, 64), (70, 64)])
@pytest.mark.parametrize("decode", [False, True])
def test_window_edge_key_dominates(nat, window, page, decode):
    """One key carries a value of 1000 and a saturated weight: the query at distance window - 1 must see it, the next
    one must not, in a prompt portion and for a single decoded token, with the key at a page border or far back."""
    T = 150
    for j in (0, page - 1, page, 2 * page + 3):
        for i in (j + window - 1, j + window):            # just inside, just outside
            if i >= T:
                continue
            cached, new = (i, 1) if decode else (max(0, i - 5), min(T, i + 3) - max(0, i - 5))
            out, ref = _attn_case(nat, 4, 2, 16, 8, window, page, [(cached, new)], spike=(0, j), seed=j)
            row = i - cached
            seen = ref[row].abs().max().item() > 500
            assert seen == (i - j < window)
            assert rel(out, ref) < 2e-5
            assert (out[row].abs().max().item() > 500) == seen


@pytest.mark.parametrize("H,G,d", [(8, 1, 64), (4, 2, 32), (4, 4, 128), (3, 1, 96)])
@pytest.mark.parametrize("window", [1, 33, 64, 65, 200, 1000])
def test_bfloat16_prompt_portions_on_the_tensor_cores(nat, H, G, d, window):
    """Prompt portions longer than one query tile and one key tile, after cached tokens, beside single tokens, in
    16-token pages: bfloat16 inputs against the plain model on the same (rounded) inputs."""
    out, ref = _attn_case(nat, H, G, d, d, window, 16, [(0, 150), (100, 90), (37, 1), (3, 67), (0, 1), (129, 2)],
                          dtype=torch.bfloat16, seed=window)
    assert rel(out, ref) < 1e-2


@pytest.mark.parametrize("window,page", [(17, 16), (64, 64), (70, 64), (129, 16)])
def test_bfloat16_window_edge_key_dominates(nat, window, page):
    T = 300
    for j in (0, page - 1, 64, 2 * page + 3):
        for i in (j + window - 1, j + window):
            for decode in (False, True):
                cached, new = (i, 1) if decode else (max(0, i - 70), min(T, i + 3) - max(0, i - 70))
                out, ref = _attn_case(nat, 4, 2, 32, 32, window, page, [(cached, new)], dtype=torch.bfloat16, spike=(0, j), seed=j)
                row = i - cached
                seen = ref[row].abs().max().item() > 500
                assert seen == (i - j < window)
                assert (out[row].float().abs().max().item() > 500) == seen
                assert rel(out, ref) < 1e-2


@pytest.mark.parametrize("m,n,k", [(1, 128, 64), (37, 256, 192), (600, 128, 64)])
def test_up_projection_with_squared_relu_epilogue(nat, m, n, k):
    """The feed-forward's first half, max(x W^T, 0)^2: activation in the GEMM epilogue for decode-sized batches, library
    GEMM + activation kernel for long portions; both against the plain model on the same bfloat16 inputs."""
    from nano_qwen3tts_vllm_b200.layers.linear import linear_relu_sq
    g = torch.Generator().manual_seed(m)
    x = torch.randn(m, k, generator=g).to(torch.bfloat16)
    w = (torch.randn(n, k, generator=g) * k ** -0.5).to(torch.bfloat16)
    got = linear_relu_sq(x.to(DEV), w.to(DEV))
    ref = O.relu_squared(x.double() @ w.double().T)
    assert got.dtype == torch.bfloat16 and rel(got, ref) < 2e-2
    assert (got.float() >= 0).all()


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-5), (torch.bfloat16, 1e-2)])
def test_far_key_among_hundreds(nat, dtype, tol):
    """A dominating key 699 or 700 positions back, behind hundreds of ordinary keys and a dozen page borders, with a
    window of 700: seen at distance 699 and not at 700, by a single decoded token, by a short portion and by a portion
    longer than a query tile that starts in the middle of the context."""
    window, page, j = 700, 64, 37
    for i in (j + window - 1, j + window):
        for cached, new in ((i, 1), (i - 1, 3), (i - 100, 130)):
            out, ref = _attn_case(nat, 4, 2, 32, 32, window, page, [(cached, new), (5, 1)], dtype=dtype, spike=(0, j), seed=i)
            row = i - cached
            seen = ref[row].abs().max().item() > 500
            assert seen == (i - j < window)
            assert (out[row].float().abs().max().item() > 500) == seen
            assert rel(out, ref) < tol


@pytest.mark.parametrize("cols,ff,n", [(72, 136, 700), (64, 40, 300), (256, 128, 5)])
def test_grouped_experts_on_the_tensor_cores(nat, cols, ff, n):
    """Groups longer than one 128-row tile, inner sizes with a tail slice, more than one column tile, a handful of rows,
    and an expert nobody chose: the grouped launch against the plain model."""
    from nano_qwen3tts_vllm_b200.layers.moe import SigmoidTopKMoE
    g = torch.Generator().manual_seed(11)
    E, top = 6, 2
    for dtype, tol in ((torch.float32, 2e-5), (torch.bfloat16, 3e-2)):
        moe = SigmoidTopKMoE(cols, ff, E, top, 0.8).to(DEV)
        router = torch.randn(E, cols, generator=g) * 0.3
        router[4] = -10.0 * torch.ones(cols)                       # h > 0 below: expert 4 is never chosen
        up = (torch.randn(E, ff, cols, generator=g) * cols ** -0.5).to(dtype)
        down = (torch.randn(E, cols, ff, generator=g) * ff ** -0.5).to(dtype)
        h = (torch.rand(n, cols, generator=g) + 0.1).to(dtype)
        moe.router.copy_(router)
        moe.up.data, moe.down.data = up.to(DEV), down.to(DEV)
        ref = O.moe_ff(h.double(), router.double(), list(up.double()), list(down.double()), top, 0.8)
        z, zw = moe(h.to(DEV))
        out = (zw.double().cpu()[:, :, None] * z.double().cpu().view(n, top, cols)).sum(1)
        assert rel(out, ref) < tol


@pytest.mark.parametrize("E,top,cols", [(5, 2, 48), (12, 3, 256), (4, 4, 40), (7, 1, 100), (70, 6, 64)])
def test_router_and_grouped_experts(nat, E, top, cols):
    from nano_qwen3tts_vllm_b200.layers.moe import SigmoidTopKMoE
    g = torch.Generator().manual_seed(E)
    n, ff = 37, 24
    for dtype, tol in ((torch.float32, 2e-5), (torch.bfloat16, 3e-2)):
        moe = SigmoidTopKMoE(cols, ff, E, top, 1.7).to(DEV)
        router = torch.randn(E, cols, generator=g) * 0.3
        up = (torch.randn(E, ff, cols, generator=g) * cols ** -0.5).to(dtype)
        down = (torch.randn(E, cols, ff, generator=g) * ff ** -0.5).to(dtype)
        h = torch.randn(n, cols, generator=g).to(dtype)
        moe.router.copy_(router)
        moe.up.data = up.to(DEV)
        moe.down.data = down.to(DEV)
        idx, w, offsets, sorted_pair = moe.route(h.to(DEV))
        ridx, rw = O.moe_route(h.double(), router.double(), top, 1.7)
        assert torch.equal(idx.cpu().long().sort(-1).values, ridx.sort(-1).values)
        order, rorder = idx.cpu().long().argsort(-1), ridx.argsort(-1)
        assert rel(w.cpu().gather(1, order), rw.gather(1, rorder)) < 1e-5
        counts = torch.bincount(idx.cpu().flatten().long(), minlength=E)
        assert torch.equal(offsets.cpu().long(), torch.cat([torch.zeros(1, dtype=torch.long), counts.cumsum(0)]))
        assert sorted(sorted_pair.cpu().tolist()) == list(range(n * top))
        z, zw = moe(h.to(DEV))
        got = (zw.double().cpu()[:, :, None] * z.double().cpu().view(n, top, cols)).sum(1)
        ref = O.moe_ff(h.double(), router.double(), list(up.double()), list(down.double()), top, 1.7)
        assert rel(got, ref) < tol


# ------------------------------------------------------------------------------------------------ through the engine
def make_engine(cfg: dict, sd: dict, dtype="float32", pages=12, page=64, seqs=4, slots=None, eager=True, budget=None):
    from nano_qwen3tts_vllm_b200.config import BokenexConfig
    from nano_qwen3tts_vllm_b200.engine.llm_engine.lm_engine import CausalLMEngine
    c = BokenexConfig.from_dict(cfg)
    return CausalLMEngine(c, state_dict={k: v.to(torch.bfloat16) for k, v in sd.items()}, dtype=dtype, kvcache_block_size=page,
                          num_kvcache_blocks=pages, max_num_seqs=seqs, max_state_slots=slots or seqs,
                          max_model_len=c.max_positions, max_num_batched_tokens=budget or seqs * c.max_positions,
                          enforce_eager=eager, device=DEV)


def replay(engine, requests: dict, schedule: list):
    """Feed ``schedule`` = [[(id, count), ...], ...] through engine.step as held sequences; logits of every position."""
    at = {i: 0 for i in requests}
    live, got = set(), {i: [] for i in requests}
    for step in schedule:
        want = {}
        for i, n in step:
            toks = requests[i][at[i]:at[i] + n]
            if i in live:
                engine.feed(i, toks)
            else:
                engine.add_request(toks, request_id=i, hold=True)
                live.add(i)
            want[i] = list(range(n))
            at[i] += n
        out = engine.step(want=want)
        assert out.scheduled == {i: n for i, n in step}
        o = 0
        for i, n in step:
            got[i].append(out.logits[o:o + n].double().cpu())
            o += n
        for i, _ in step:
            if at[i] == len(requests[i]):
                engine.clear_request(i)
                live.discard(i)
    return {i: torch.cat(v) for i, v in got.items() if v}


def nerr(got, ref):
    """Per-position error: rms over the vocabulary of the mean-free difference, relative to the rms of the logits."""
    d = got - ref
    d = d - d.mean(-1, keepdim=True)
    return (d.pow(2).mean(-1).sqrt() / ref.pow(2).mean().sqrt()).max().item()


def nerr_rows(got, ref):
    d = got - ref
    d = d - d.mean(-1, keepdim=True)
    return d.pow(2).mean(-1).sqrt() / ref.pow(2).mean().sqrt()


def tokens_for(cfg, n, seed):
    return torch.randint(0, cfg["vocab"], (n,), generator=torch.Generator().manual_seed(seed)).tolist()


CONFIGS = {
    "mixed_kinds": dict(),
    "one_kv_head_no_conv": dict(kv_heads=1, taps=1, window=1, residual_mult=1.0, kinds=("moe", "dense")),
    "all_heads_own_kv_top1": dict(heads=3, kv_heads=3, taps=2, top=1, experts=3, dim=16, vdim=8, kinds=("moe", None)),
    "every_expert_chosen": dict(experts=4, top=4, taps=5, window=70, kinds=("moe",), n_layers=2, max_positions=200),
    "tensor_core_shapes": dict(width=128, heads=4, kv_heads=2, dim=32, vdim=32, ff=128, expert_ff=64, window=20,
                               kinds=("dense", "moe"), n_layers=2, vocab=128),
}


@pytest.mark.parametrize("name", list(CONFIGS))
def test_whole_prompt_decode_and_portions_match_plain_model(name):
    cfg = O.random_config(1, **CONFIGS[name])
    sd = O.random_weights(cfg, seed=3)
    T = cfg["max_positions"] - 6
    toks = tokens_for(cfg, T, 5)
    ref = O.forward(cfg, sd, toks)
    eng = make_engine(cfg, sd)
    try:
        whole = replay(eng, {"a": toks}, [[("a", T)]])["a"]
        assert nerr(whole, ref) < 2e-5
        one_by_one = replay(eng, {"b": toks}, [[("b", 1)] for _ in range(T)])["b"]
        assert nerr(one_by_one, ref) < 2e-5
        cuts, left = [], T
        for n in [2, 3, 1, 17, 2, 1, 1, 30, 2]:
            n = min(n, left)
            if n:
                cuts.append(n)
                left -= n
        cuts += [1] * left
        portions = replay(eng, {"c": toks}, [[("c", n)] for n in cuts])["c"]
        assert nerr(portions, ref) < 2e-5
    finally:
        eng.exit()


def test_unequal_batch_matches_each_alone_and_reuses_pages_and_slots():
    """Four live requests of different lengths in one pool of 6 pages of 16 tokens and 2 state slots... requests end and
    new ones take over their pages and slots in the middle of other requests' prompts."""
    cfg = O.random_config(2, max_positions=80, window=20, taps=4)
    sd = O.random_weights(cfg, seed=4)
    req = {i: tokens_for(cfg, n, 10 + k) for k, (i, n) in enumerate([("a", 40), ("b", 9), ("c", 33), ("d", 1), ("e", 30)])}
    ref = {i: O.forward(cfg, sd, t) for i, t in req.items()}
    eng = make_engine(cfg, sd, pages=6, page=16, seqs=2, slots=2)
    try:
        schedule = [[("a", 7), ("b", 2)], [("a", 2), ("b", 1)], [("b", 6)],                      # b ends: slot + page free
                    [("a", 20), ("c", 5)], [("c", 2), ("a", 1)], [("a", 10)],                    # a ends: 3 pages free
                    [("c", 26), ("d", 1)],                                                       # d ends at once
                    [("e", 13)], [("e", 1)], [("e", 16)]]
        got = replay(eng, req, schedule)
        for i in req:
            assert got[i].shape == ref[i].shape
            assert nerr(got[i], ref[i]) < 2e-5, i
        assert len(eng.scheduler.block_manager.free_block_ids) == 6 and eng.scheduler.state_slots.available() == 2
    finally:
        eng.exit()


def test_long_decode_over_pages_and_windows_graph_equals_eager():
    cfg = O.random_config(3, max_positions=230, window=37, taps=4, n_layers=3)
    sd = O.random_weights(cfg, seed=6)
    req = {"a": tokens_for(cfg, 225, 1), "b": tokens_for(cfg, 140, 2)}
    ref = {i: O.forward(cfg, sd, t) for i, t in req.items()}
    sched = [[("a", 60), ("b", 3)]] + [[("a", 1), ("b", 1)] for _ in range(137)] + [[("a", 1)] for _ in range(28)]
    outs = []
    for eager in (True, False):
        eng = make_engine(cfg, sd, pages=7, page=64, seqs=3, eager=eager)
        try:
            got = replay(eng, req, sched)
            assert eager or eng.model_runner.graphs
        finally:
            eng.exit()
        for i in req:
            assert nerr(got[i], ref[i]) < 2e-5, (i, eager)
        outs.append(got)
    for i in req:
        assert torch.equal(outs[0][i], outs[1][i])


def test_bfloat16_serving_precision_and_cut_independence():
    cfg = O.random_config(4, **CONFIGS["tensor_core_shapes"])
    sd = O.random_weights(cfg, seed=8)
    T = 90
    toks = tokens_for(cfg, T, 3)
    ref = O.forward(cfg, sd, toks)
    eng = make_engine(cfg, sd, dtype="bfloat16", eager=False)
    try:
        whole = replay(eng, {"a": toks}, [[("a", T)]])["a"]
        cut = replay(eng, {"b": toks}, [[("b", 50)], [("b", 2)]] + [[("b", 1)]] * 38)["b"]
    finally:
        eng.exit()
    # bfloat16 rounding can flip a close router decision at a few positions (a different expert: a large difference
    # there); everywhere else the error is rounding noise
    for got, want in ((whole, ref), (cut, ref), (cut, whole)):
        e = nerr_rows(got, want)
        assert e.median().item() < 0.03 and (e > 0.1).float().mean().item() < 0.1, e


@pytest.mark.parametrize("dtype,tol", [("float32", 2e-5), ("bfloat16", None)])
def test_sizes_that_fit_no_vector_width(dtype, tol):
    """Width, head sizes, inner sizes and vocabulary that are multiples of 2 only (no 16-byte rows anywhere), five heads
    that each own their key/value head, two taps, one expert of three: every kernel takes its general path."""
    cfg = O.random_config(7, width=50, vocab=41, heads=5, kv_heads=5, dim=6, vdim=10, ff=42, expert_ff=22, experts=3, top=1,
                          taps=2, window=13, kinds=("moe", "dense", None), n_layers=3, max_positions=80)
    sd = O.random_weights(cfg, seed=4)
    toks = tokens_for(cfg, 70, 5)
    ref = O.forward(cfg, sd, toks)
    eng = make_engine(cfg, sd, dtype=dtype, pages=3, page=64, seqs=2)
    try:
        whole = replay(eng, {"a": toks}, [[("a", 70)]])["a"]
        cut = replay(eng, {"b": toks}, [[("b", 31)], [("b", 2)], [("b", 17)]] + [[("b", 1)]] * 20)["b"]
    finally:
        eng.exit()
    if tol is not None:
        assert nerr(whole, ref) < tol and nerr(cut, ref) < tol
    else:
        for got, want in ((whole, ref), (cut, ref), (cut, whole)):
            e = nerr_rows(got, want)
            assert e.median().item() < 0.03 and (e > 0.1).float().mean().item() < 0.1, e


def test_bfloat16_wide_group_mixed_batch_equals_each_alone():
    """Six query heads on one key/value head of 64, window shorter than the prompts, bfloat16 with CUDA graphs: a batch
    that mixes portions and decoded tokens of three requests over reused pages and slots gives each request the
    logits it gets alone (rounding apart) and stays close to the plain model."""
    cfg = O.random_config(6, width=128, heads=12, kv_heads=2, dim=64, vdim=64, ff=128, expert_ff=64, window=37, taps=4,
                          kinds=("dense", "moe"), n_layers=2, vocab=96, max_positions=160)
    sd = O.random_weights(cfg, seed=12)
    req = {"a": tokens_for(cfg, 120, 1), "b": tokens_for(cfg, 75, 2), "c": tokens_for(cfg, 60, 3)}
    ref = {i: O.forward(cfg, sd, t) for i, t in req.items()}
    eng = make_engine(cfg, sd, dtype="bfloat16", eager=False, pages=5, page=64, seqs=2, slots=2)
    try:
        alone = {i: replay(eng, {i: t}, [[(i, len(t) - 20)]] + [[(i, 1)]] * 20)[i] for i, t in req.items()}
        sched = [[("a", 70)], [("a", 30), ("b", 40)]] + [[("a", 1), ("b", 7)]] * 5 + [[("a", 1)]] * 15     # a ends: 120
        sched += [[("c", 33)], [("c", 2)]] + [[("c", 1)]] * 25                                              # c reuses a's pages
        mixed = replay(eng, {"a": req["a"], "b": req["b"], "c": req["c"]}, sched)
        assert len(eng.scheduler.block_manager.free_block_ids) == 5 and eng.scheduler.state_slots.available() == 2
    finally:
        eng.exit()
    for i in req:
        for got, want in ((alone[i], ref[i]), (mixed[i], ref[i]), (mixed[i], alone[i])):
            e = nerr_rows(got, want)
            assert e.median().item() < 0.03 and (e > 0.1).float().mean().item() < 0.1, (i, e)


def test_greedy_generation_through_the_scheduler():
    """``generate`` with top_k = 1: prompts of unequal length, a token budget that cuts the prompts into portions, fewer
    state slots than requests (the rest wait).  Every generated token must be the plain model's argmax, or lie within
    float32 noise of it."""
    from nano_qwen3tts_vllm_b200.sampling_params import SamplingParams
    cfg = O.random_config(5, max_positions=64, window=11)
    sd = O.random_weights(cfg, seed=9)
    prompts = [tokens_for(cfg, n, 20 + n) for n in (17, 3, 29, 1, 8)]
    eng = make_engine(cfg, sd, pages=8, page=16, seqs=3, slots=3, budget=64)
    eng.scheduler.max_num_batched_tokens = 12
    try:
        outs = eng.generate(prompts, SamplingParams(temperature=1.0, max_tokens=9, top_k=1, ignore_eos=True))
        assert len(eng.scheduler.block_manager.free_block_ids) == 8 and eng.scheduler.state_slots.available() == 3
    finally:
        eng.exit()
    for p, o in zip(prompts, outs):
        gen = o["token_ids"]
        assert len(gen) == 9
        logits = O.forward(cfg, sd, p + gen)
        for k, t in enumerate(gen):
            row = logits[len(p) + k - 1]
            assert row[t] >= row.max() - 1e-4 * row.abs().max()
