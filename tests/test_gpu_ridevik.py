"""Ridevik on the GPU against the plain float64 restatement in ``oracle/ridevik.py`` (no code shared with the package).

Kernel level: every mechanism alone, with inputs built so that a fault shows (one key that takes the whole softmax,
placed just inside / just outside a window, at a page border, far back; a sink that swallows a head; a token-shift row
carried over portions of 1, 2, 3 tokens through a slot another sequence used).  Engine level, through ``CausalLMEngine``
and its scheduler: whole prompts, token-by-token decoding, portions, mixed batches, reuse of pages and state slots, long
decoding across pages and windows, layers that share weights, odd sizes, greedy generation, CUDA graphs against eager.
The float32 engine is the sharp comparison; bfloat16 is checked against its rounding noise."""
import math

import pytest
import torch

from oracle import ridevik as O

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
@pytest.mark.parametrize("cols,groups", [(40, 1), (40, 5), (256, 2), (1000, 8), (9000, 3)])
def test_embedding_group_norm_residual_and_activations(nat, dtype, cols, groups):
    g = torch.Generator().manual_seed(cols)
    n, vocab, top, eps = 6, 19, 3, 1e-3
    tol = 1e-5 if dtype == torch.float32 else 1e-2
    emb = torch.randn(vocab, cols, generator=g).to(dtype)
    tok = torch.randint(0, vocab, (n,), generator=g).int()
    x = torch.empty(n, cols, device=DEV)
    nat.embed_scale(tok.to(DEV), emb.to(DEV), 2.5, x)
    x_ref = emb.double()[tok.long()] * 2.5
    assert rel(x, x_ref) < 1e-6
    w = torch.rand(cols, generator=g) + 0.5
    a = torch.randn(n, cols, generator=g).to(dtype)
    z = torch.randn(n * top, cols, generator=g).to(dtype)
    zw = torch.rand(n, top, generator=g)
    for use_a, use_z, copy in [(1, 0, True), (0, 1, False), (1, 1, True)]:
        xx = x_ref.float().to(DEV)
        cp = torch.empty(n, cols, dtype=dtype, device=DEV) if copy else None
        nat.group_norm_residual(xx, a.to(DEV) if use_a else None, z.to(DEV) if use_z else None, zw.to(DEV) if use_z else None,
                                w.to(DEV), groups, eps, cp, dtype)
        y = use_a * a.double() + use_z * (zw.double()[:, :, None] * z.double().view(n, top, cols)).sum(1)
        ref = x_ref.float().double() + O.grouped_rms_norm(y, w.double(), eps, groups)
        assert rel(xx, ref) < 1e-5
        if copy:
            assert rel(cp, ref) < tol
    rows = torch.tensor([4, 0, 4], dtype=torch.int32)
    out = nat.gather_group_norm(x, rows.to(DEV), w.to(DEV), groups, eps, dtype)
    assert rel(out, O.grouped_rms_norm(x_ref[rows.long()], w.double(), eps, groups)) < tol
    # activations: both branches of xIELU with and without bias; the gated SiLU product
    y = (3 * torch.randn(5, 34, generator=g)).to(dtype)
    b = torch.randn(34, generator=g).to(dtype)
    for pq in ([0.3, -0.8], [-2.0, 1.5]):
        p = torch.tensor(pq)
        assert rel(nat.xielu_(y.clone().to(DEV), b.to(DEV), p.to(DEV)), O.xielu(y.double() + b.double(), p[0].double(), p[1].double())) < tol
        assert rel(nat.xielu_(y.clone().to(DEV), None, p.to(DEV)), O.xielu(y.double(), p[0].double(), p[1].double())) < tol
    gu = torch.randn(7, 2 * 22, generator=g).to(dtype)
    ref = torch.nn.functional.silu(gu.double()[:, :22]) * gu.double()[:, 22:]
    assert rel(nat.silu_mul(gu.to(DEV)), ref) < tol


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("D", [70, 72, 1028])
def test_token_shift_in_portions_through_a_reused_slot(nat, dtype, D):
    """Two sequences cut into portions of 1, 2, 3, 7 ... tokens; their previous rows travel through state slots that
    hold another owner's rows at the start (position 0 must read zero all the same)."""
    g = torch.Generator().manual_seed(5)
    T = 33
    xs = [torch.randn(T, D, generator=g), torch.randn(T, D, generator=g)]
    mu = torch.rand(D, generator=g)
    state = torch.full((3, D), 9.0, device=DEV)
    got = [[], []]
    at = 0
    for n in [1, 2, 3, 7, 1, 1, 12, 2, 4]:
        lay = Lay([(at, n, 2, [0, 1, 2]), (at, n, 0, [3, 4, 5])], 16, 3)
        x = torch.cat([xs[0][at:at + n], xs[1][at:at + n]]).to(DEV)
        out = torch.empty(2 * n, D, dtype=dtype, device=DEV)
        nat.token_shift(x, mu.to(DEV), state, lay, out)
        got[0].append(out[:n].cpu()), got[1].append(out[n:].cpu())
        at += n
    assert at == T
    for s in range(2):
        assert rel(torch.cat(got[s]), O.token_shift(xs[s].double(), mu.double())) < (1e-6 if dtype == torch.float32 else 1e-2)
    assert torch.equal(state[2].cpu(), xs[0][-1]) and torch.equal(state[0].cpu(), xs[1][-1]) and bool((state[1] == 9.0).all())


@pytest.mark.parametrize("q_rank,kv_rank,rot_dim,rot_dims,scaling", [(12, 24, 8, 8, True), (0, 16, 6, 4, False), (40, 200, 34, 34, True)])
def test_latent_preparation_norms_rotation_and_cache_rows(nat, q_rank, kv_rank, rot_dim, rot_dims, scaling):
    g = torch.Generator().manual_seed(kv_rank)
    page, eps, extra = 16, 1e-4, 5
    sc = {"factor": 3.0, "original": 16, "fast": 4.0, "slow": 0.5} if scaling else None
    from nano_qwen3tts_vllm_b200.layers.rotary_embedding import PairRotary
    rot = PairRotary(rot_dims, 300.0, sc).to(DEV)
    f_ref, mult_ref = O.rotary_frequencies(rot_dims, 300.0, sc)
    assert rel(rot.freq, f_ref) < 1e-6 and abs(rot.mult - mult_ref) < 1e-12
    seqs = [(37, 11, 0, [4, 1, 6]), (0, 3, 1, [2]), (1000, 1, 2, [0] * 62 + [5])]
    lay = Lay(seqs, page, 63)
    n = lay.n_tokens
    u = torch.randn(n, extra + q_rank + kv_rank + rot_dim + 3, generator=g)
    wq, wkv = torch.rand(max(q_rank, 1), generator=g) + 0.5, torch.rand(kv_rank, generator=g) + 0.5
    cache = torch.zeros(7, page, kv_rank + rot_dim, device=DEV)
    cq = torch.empty(n, q_rank, device=DEV) if q_rank else None
    nat.latent_prep(u.to(DEV), extra, extra + q_rank, cq, wq.to(DEV) if q_rank else None, wkv.to(DEV), rot.freq, rot.mult, lay, cache,
                    q_rank, kv_rank, rot_dim, rot_dims, eps)
    ud = u.double()
    if q_rank:
        assert rel(cq, O.rms_norm(ud[:, extra:extra + q_rank], wq.double(), eps)) < 1e-5
    pos = lay.positions.cpu().long()
    c_ref = O.rms_norm(ud[:, extra + q_rank:extra + q_rank + kv_rank], wkv.double(), eps)
    kr_ref = O.rotate_pairs(ud[:, extra + q_rank + kv_rank:extra + q_rank + kv_rank + rot_dim], pos, f_ref, mult_ref, rot_dims)
    rows = cache.view(-1, kv_rank + rot_dim)[lay.slot_mapping.long()].cpu()
    assert rel(rows[:, :kv_rank], c_ref) < 1e-5
    # the angle position * f is formed in float: at position 1000 it is good to ~1e-4 rad
    assert rel(rows[:, kv_rank:], kr_ref) < 2e-4
    assert rel(rows[:14, kv_rank:], kr_ref[:14]) < 1e-5


def _attn_case(nat, H, r, dr, window, page, seqs, dtype=torch.float32, spike=None, sink_big=None, seed=0, path=0, rot_dims=None,
               splits=None):
    """seqs: [(cached tokens, new tokens)].  Fills the cache with the sequences' rows, runs the kernel for the new
    tokens, compares with the plain implementation over the whole sequence.  ``spike`` = (sequence, key position): that
    key's score exceeds every other by a wide margin for every query.  ``sink_big``: head whose sink swallows the softmax."""
    from nano_qwen3tts_vllm_b200.layers.rotary_embedding import PairRotary
    g = torch.Generator().manual_seed(seed)
    rot_dims = dr if rot_dims is None else rot_dims
    rot = PairRotary(rot_dims, 50.0, None).to(DEV)
    f_ref, _ = O.rotary_frequencies(rot_dims, 50.0, None)
    nb = [math.ceil((c + n) / page) for c, n in seqs]
    perm = torch.randperm(sum(nb) + 3, generator=g).tolist()
    tables, o = [], 0
    for k in nb:
        tables.append(perm[o:o + k])
        o += k
    cache = torch.zeros(sum(nb) + 3, page, r + dr, dtype=dtype, device=DEV)
    flat = cache.view(-1, r + dr)
    scale = 0.3
    sink = torch.randn(H, generator=g)
    if sink_big is not None:
        sink[sink_big] = 60.0
    C, KR, QL, QR = [], [], [], []
    for s, (c, n) in enumerate(seqs):
        T = c + n
        lat = torch.randn(T, r, generator=g).to(dtype)
        kr = torch.randn(T, dr, generator=g).to(dtype)
        ql = torch.randn(T, H, r, generator=g).to(dtype)
        qr = torch.randn(T, H, dr, generator=g).to(dtype)
        if spike is not None and spike[0] == s:
            ql[:, :, 0] = 6.0                                   # every query looks along coordinate 0 ...
            lat[:, 0] = 0.0
            lat[spike[1], 0] = 40.0                             # ... where only the spiked key has anything
            lat[spike[1], 1:] *= 5.0
        slots = torch.tensor([tables[s][p // page] * page + p % page for p in range(T)])
        flat[slots.to(DEV)] = torch.cat([lat, kr], 1).to(DEV)
        C.append(lat), KR.append(kr), QL.append(ql), QR.append(qr)
    lay = Lay([(c, n, 0, tables[s]) for s, (c, n) in enumerate(seqs)], page, max(nb))
    n_new = lay.n_tokens
    ql = torch.cat([QL[s][c:] for s, (c, n) in enumerate(seqs)]).transpose(0, 1).contiguous().to(DEV)        # [H, n, r]
    qr = torch.cat([QR[s][c:] for s, (c, n) in enumerate(seqs)]).contiguous().to(DEV)                        # [n, H, dr]
    out = torch.full((H, n_new, r), 7.0, dtype=dtype, device=DEV)
    nat.latent_attn(ql, (r, n_new * r), qr, (H * dr, dr), cache, out, (r, n_new * r), sink.to(DEV), rot.freq, 1.0, rot_dims, lay,
                    H, r, dr, page, window, scale, path, splits_override=splits)
    got = out.transpose(0, 1).cpu()
    o = 0
    worst = 0.0
    for s, (c, n) in enumerate(seqs):
        T = c + n
        qrr = O.rotate_pairs(QR[s].double().transpose(0, 1), torch.arange(T), f_ref, 1.0, rot_dims).transpose(0, 1)
        q = torch.cat([QL[s].double(), qrr], -1)
        k = torch.cat([C[s].double(), KR[s].double()], -1)[:, None, :].expand(T, H, r + dr)
        v = C[s].double()[:, None, :].expand(T, H, r)
        ref = O.sink_softmax_attention(q, k, v, scale, window or None, sink.double())[c:]
        worst = max(worst, ((got[o:o + n].double() - ref).abs().max() / ref.abs().max().clamp_min(1e-3)).item())
        o += n
    return worst


@pytest.mark.parametrize("H,r,dr", [(3, 24, 8), (8, 64, 24), (5, 40, 6), (16, 128, 16)])
@pytest.mark.parametrize("window", [0, 1, 7, 64, 65])
def test_latent_attention_prompts_portions_and_decoded_tokens_in_one_launch(nat, H, r, dr, window):
    seqs = [(0, 70), (50, 19), (129, 1), (64, 1), (0, 1), (63, 2)]
    assert _attn_case(nat, H, r, dr, window, 16, seqs, seed=H + window) < 2e-5
    assert _attn_case(nat, H, r, dr, window, 64, seqs, seed=H + window + 1, rot_dims=dr - 2) < 2e-5


@pytest.mark.parametrize("H,r,dr", [(8, 64, 16), (4, 96, 8), (16, 128, 16), (3, 32, 8), (20, 64, 8), (2, 256, 64), (1, 160, 24)])
@pytest.mark.parametrize("window", [0, 1, 7, 64, 65, 130])
def test_tensor_core_latent_attention_against_plain_model_and_plain_kernel(nat, H, r, dr, window):
    """The bfloat16 tensor-core kernel (forced) on mixed steps: tiles of several tokens (fewer than 16 heads), of one
    token (16 heads), several head blocks (20 heads), rows of different sequences, keys across many 64-key tiles."""
    seqs = [(0, 70), (50, 19), (129, 1), (64, 1), (0, 1), (63, 2), (200, 37)]
    for page, rd in ((16, None), (64, dr - 2)):
        for path in (nat.LATENT_ATTN_TENSOR, nat.LATENT_ATTN_TENSOR_SHARED, nat.LATENT_ATTN_PLAIN, nat.LATENT_ATTN_AUTO):
            e = _attn_case(nat, H, r, dr, window, page, seqs, dtype=torch.bfloat16, seed=H + window, path=path, rot_dims=rd)
            assert e < 2e-2, (path, e)


@pytest.mark.parametrize("H,r,dr", [(8, 64, 16), (4, 96, 24), (20, 64, 8)])
@pytest.mark.parametrize("window", [0, 70, 300])
def test_decode_steps_whose_keys_are_cut_into_ranges_and_merged(nat, H, r, dr, window):
    """A decode step on the tensor-core kernel with each sequence's keys cut into 2, 3 or 8 ranges (more ranges than some
    sequences have key tiles: empty ranges; the sink must count once), also with a spiked key in the last or first range."""
    seqs = [(400, 1), (63, 1), (0, 1), (64, 1), (129, 1), (777, 1)]
    for splits in (None, 2, 3, 8):
        assert _attn_case(nat, H, r, dr, window, 64, seqs, dtype=torch.bfloat16, seed=H, path=nat.LATENT_ATTN_TENSOR, splits=splits) < 2e-2
    for sp in ((0, 399), (0, 5), (5, 500), (5, 776)):
        assert _attn_case(nat, H, r, dr, window, 16, seqs, dtype=torch.bfloat16, seed=H, path=nat.LATENT_ATTN_TENSOR, splits=3, spike=sp) < 2e-2
    assert _attn_case(nat, H, r, dr, window, 16, [(100, 9), (300, 40)], dtype=torch.bfloat16, seed=1, path=nat.LATENT_ATTN_TENSOR, splits=2) < 2e-2
    assert _attn_case(nat, H, r, dr, 0, 16, seqs, dtype=torch.bfloat16, seed=2, path=nat.LATENT_ATTN_TENSOR, splits=4, sink_big=1) < 2e-2


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-5), (torch.bfloat16, 2e-2)])
@pytest.mark.parametrize("page", [16, 64])
@pytest.mark.parametrize("window", [33, 64, 200])
def test_one_key_that_takes_the_softmax_at_window_edges_and_page_borders(nat, dtype, tol, page, window):
    """The spiked key at position p is seen by queries p .. p + window - 1 and by no later one; p sits on the last slot
    of a page, the first of the next, and mid-page; queries are prompt rows of a portion and single decoded tokens."""
    H, r, dr = 4, 32, 16
    for p in (page - 1, page, 2 * page + 5):
        for q_first in (p + window - 3, p + window - 1, p + window):           # a portion that straddles the edge
            seqs = [(q_first, 6), (p + window - 1, 1), (p + window, 1), (p, 1), (0, p + 2)]
            spikes = [(0, p), (1, p), (2, p), (3, p), (4, p)]
            for sp in spikes:
                assert _attn_case(nat, H, r, dr, window, page, seqs, dtype=dtype, spike=sp, seed=p) < tol, (p, q_first, sp)


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-5), (torch.bfloat16, 2e-2)])
def test_far_key_among_hundreds_and_a_sink_that_swallows_a_head(nat, dtype, tol):
    H, r, dr = 8, 64, 16
    for window, back in [(0, 899), (700, 699), (700, 700)]:
        seqs = [(900, 1), (880, 21)]
        assert _attn_case(nat, H, r, dr, window, 64, seqs, dtype=dtype, spike=(0, 900 - back), seed=back) < tol
        assert _attn_case(nat, H, r, dr, window, 64, seqs, dtype=dtype, spike=(1, 900 - back), seed=back + 1) < tol
    assert _attn_case(nat, H, r, dr, 0, 16, [(0, 40), (39, 1)], dtype=dtype, sink_big=3, seed=2) < tol


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("E,top,n", [(5, 2, 37), (4, 4, 9), (7, 1, 300), (12, 3, 1)])
def test_softmax_over_chosen_router_with_bias_and_gated_experts(nat, dtype, E, top, n):
    from nano_qwen3tts_vllm_b200.layers.moe import SoftmaxTopKGatedMoE
    g = torch.Generator().manual_seed(E * 10 + top)
    cols, ff = 48, 24
    tol = 2e-5 if dtype == torch.float32 else 3e-2
    h = torch.randn(n, cols, generator=g).to(dtype)
    p = {"router": torch.randn(E, cols, generator=g).to(torch.bfloat16), "router.b": (2 * torch.randn(E, generator=g)).to(torch.bfloat16)}
    if E == 5:
        p["router.b"][3] = -50.0                                                 # an expert nobody chooses
    for e in range(E):
        p[f"e{e}.gate"] = (torch.randn(ff, cols, generator=g) * cols ** -0.5).to(dtype)
        p[f"e{e}.up"] = (torch.randn(ff, cols, generator=g) * cols ** -0.5).to(dtype)
        p[f"e{e}.down"] = (torch.randn(cols, ff, generator=g) * ff ** -0.5).to(dtype)
    with torch.device(DEV):
        prev = torch.get_default_dtype()
        torch.set_default_dtype(dtype)
        try:
            moe = SoftmaxTopKGatedMoE(cols, ff, E, top)
        finally:
            torch.set_default_dtype(prev)
    moe.router.data = p["router"].float().to(DEV)
    moe.router_bias.data = p["router.b"].float().to(DEV)
    moe.up.data = torch.stack([torch.cat([p[f"e{e}.gate"], p[f"e{e}.up"]]) for e in range(E)]).to(DEV)
    moe.down.data = torch.stack([p[f"e{e}.down"] for e in range(E)]).to(DEV)
    idx, w, offsets, sorted_pair = moe.route(h.to(DEV))
    logits = h.double() @ p["router"].double().T + p["router.b"].double()
    val, ridx = torch.topk(logits, top, dim=-1)
    assert torch.equal(idx.cpu().long(), ridx)                                   # in descending order of the logits
    assert rel(w, torch.softmax(val, -1)) < 1e-5
    counts = torch.bincount(idx.cpu().flatten().long(), minlength=E)
    assert torch.equal(offsets.cpu().long(), torch.cat([torch.zeros(1, dtype=torch.long), counts.cumsum(0)]))
    z, zw = moe(h.to(DEV))
    got = (zw.double().cpu()[:, :, None] * z.double().cpu().view(n, top, cols)).sum(1)
    assert rel(got, O.softmax_topk_moe(h.double(), {k: v.double() for k, v in p.items()}, E, top)) < tol


# ------------------------------------------------------------------------------------------------ through the engine
def make_engine(cfg: dict, sd: dict, dtype="float32", pages=12, page=64, seqs=4, slots=None, eager=True, budget=None, max_len=256):
    from nano_qwen3tts_vllm_b200.config import RidevikConfig
    from nano_qwen3tts_vllm_b200.engine.llm_engine.lm_engine import CausalLMEngine
    c = RidevikConfig.from_dict(cfg)
    return CausalLMEngine(c, state_dict={k: v.to(torch.bfloat16) for k, v in sd.items()}, dtype=dtype, kvcache_block_size=page,
                          num_kvcache_blocks=pages, max_num_seqs=seqs, max_state_slots=slots or seqs, max_model_len=max_len,
                          max_num_batched_tokens=budget or seqs * max_len, enforce_eager=eager, device=DEV)


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


def nerr_rows(got, ref):
    """Per-position error: rms over the vocabulary of the mean-free difference, relative to the rms of the logits."""
    d = got - ref
    d = d - d.mean(-1, keepdim=True)
    return d.pow(2).mean(-1).sqrt() / ref.pow(2).mean().sqrt()


def nerr(got, ref):
    return nerr_rows(got, ref).max().item()


def tokens_for(cfg, n, seed):
    return torch.randint(0, cfg["vocab"], (n,), generator=torch.Generator().manual_seed(seed)).tolist()


def bf16_close(got, want):
    # bfloat16 rounding can flip a close router decision at a few positions (a different expert: a large difference
    # there); everywhere else the error is rounding noise
    e = nerr_rows(got, want)
    return e.median().item() < 0.03 and (e > 0.12).float().mean().item() < 0.1


CONFIGS = {
    "both_mixers_all_feed_forwards": dict(),
    "shared_layers": dict(n_layers=5, share={2: 0, 3: 1, 4: 1}, kinds=("moe", "dense")),
    "one_group_one_head_top1_window1": dict(groups=1, heads=(1, 1), top=1, window=1, kinds=("moe",), n_layers=2, scaling=False),
    "every_expert_chosen_part_rotation": dict(experts=3, top=3, rot_dim=(8, 6), rot_dims=(4, 2), groups=4, window=40,
                                              kinds=("moe", "dense"), n_layers=2, embedding_scale=1.0),
    "window_only_layers": dict(types=("latent_attention",), window=17, n_layers=2, kinds=(None, "dense")),
    "causal_only_layers": dict(types=("latent_attention_2",), n_layers=2, kinds=("dense", None)),
    "tensor_core_shapes": dict(width=128, heads=(4, 2), dim=(32, 16), rot_dim=(16, 24), vdim=(32, 48), kv_rank=(128, 96), q_rank=32,
                               ff=128, expert_ff=64, window=20, kinds=("dense", "moe"), n_layers=2, vocab=128),
}


@pytest.mark.parametrize("name", list(CONFIGS))
def test_whole_prompt_decode_and_portions_match_plain_model(name):
    cfg = O.random_config(1, **CONFIGS[name])
    sd = O.random_weights(cfg, seed=3)
    T = 90
    toks = tokens_for(cfg, T, 5)
    ref = O.forward(sd, cfg, toks)
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


def test_residual_stream_after_every_layer_run():
    cfg = O.random_config(2, n_layers=4, share={3: 1})
    sd = O.random_weights(cfg, seed=5)
    toks = tokens_for(cfg, 21, 1)
    want = []
    O.forward(sd, cfg, toks, layers_out=want)
    eng = make_engine(cfg, sd)
    try:
        eng.model_runner.model.trace_layers = got = []
        replay(eng, {"a": toks}, [[("a", 21)]])
    finally:
        eng.exit()
    assert len(got) == len(want) == 4
    for a, b in zip(got, want):
        assert rel(a, b) < 1e-5


def test_unequal_batch_matches_each_alone_and_reuses_pages_and_slots():
    """Live requests of different lengths in one pool of 6 pages of 16 tokens and 2 state slots: requests end and new
    ones take over their pages and slots in the middle of other requests' prompts."""
    cfg = O.random_config(2, window=20, share={3: 1})
    sd = O.random_weights(cfg, seed=4)
    req = {i: tokens_for(cfg, n, 10 + k) for k, (i, n) in enumerate([("a", 40), ("b", 9), ("c", 33), ("d", 1), ("e", 30)])}
    ref = {i: O.forward(sd, cfg, t) for i, t in req.items()}
    eng = make_engine(cfg, sd, pages=6, page=16, seqs=2, slots=2, max_len=80)
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
    cfg = O.random_config(3, window=37, n_layers=3, kinds=("moe", "dense", "moe"))
    sd = O.random_weights(cfg, seed=6)
    req = {"a": tokens_for(cfg, 225, 1), "b": tokens_for(cfg, 140, 2)}
    ref = {i: O.forward(sd, cfg, t) for i, t in req.items()}
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
    T = 150
    toks = tokens_for(cfg, T, 3)
    ref = O.forward(sd, cfg, toks)
    eng = make_engine(cfg, sd, dtype="bfloat16", eager=False)
    try:
        whole = replay(eng, {"a": toks}, [[("a", T)]])["a"]
        cut = replay(eng, {"b": toks}, [[("b", 50)], [("b", 2)], [("b", 60)]] + [[("b", 1)]] * 38)["b"]
    finally:
        eng.exit()
    for got, want in ((whole, ref), (cut, ref), (cut, whole)):
        assert bf16_close(got, want), nerr_rows(got, want)


@pytest.mark.parametrize("dtype,tol", [("float32", 2e-5), ("bfloat16", None)])
def test_sizes_that_fit_no_vector_width(dtype, tol):
    """Width, head sizes, ranks, inner sizes and vocabulary that are multiples of 2 only (no 16-byte rows anywhere), value
    size different from the key size, five heads, one expert of three: every kernel takes its general path."""
    cfg = O.random_config(7, width=50, vocab=41, heads=(5, 3), dim=(6, 10), rot_dim=(6, 2), vdim=(10, 6), kv_rank=(14, 22), q_rank=10,
                          ff=42, expert_ff=22, experts=3, top=1, window=13, groups=5, kinds=("moe", "dense", None), n_layers=3)
    sd = O.random_weights(cfg, seed=4)
    toks = tokens_for(cfg, 70, 5)
    ref = O.forward(sd, cfg, toks)
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
            assert bf16_close(got, want), nerr_rows(got, want)


def test_bfloat16_mixed_batch_equals_each_alone():
    """bfloat16 with CUDA graphs, a window shorter than the prompts: a batch that mixes portions and decoded tokens of
    three requests over reused pages and slots gives each request the logits it gets alone (rounding apart)."""
    cfg = O.random_config(6, width=128, heads=(16, 4), dim=(32, 32), rot_dim=(32, 16), vdim=(32, 32), kv_rank=(128, 96), q_rank=64,
                          ff=128, expert_ff=64, window=37, kinds=("dense", "moe"), n_layers=2, vocab=96)
    sd = O.random_weights(cfg, seed=12)
    req = {"a": tokens_for(cfg, 120, 1), "b": tokens_for(cfg, 75, 2), "c": tokens_for(cfg, 60, 3)}
    ref = {i: O.forward(sd, cfg, t) for i, t in req.items()}
    eng = make_engine(cfg, sd, dtype="bfloat16", eager=False, pages=5, page=64, seqs=2, slots=2, max_len=192)
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
            assert bf16_close(got, want), (i, nerr_rows(got, want))


def test_greedy_generation_through_the_scheduler():
    """``generate`` with top_k = 1: prompts of unequal length, a token budget that cuts the prompts into portions, fewer
    state slots than requests (the rest wait).  Every generated token must be the plain model's argmax, or lie within
    float32 noise of it."""
    from nano_qwen3tts_vllm_b200.sampling_params import SamplingParams
    cfg = O.random_config(5, window=11, share={2: 0})
    sd = O.random_weights(cfg, seed=9)
    prompts = [tokens_for(cfg, n, 20 + n) for n in (17, 3, 29, 1, 8)]
    eng = make_engine(cfg, sd, pages=8, page=16, seqs=3, slots=3, budget=64, max_len=64)
    eng.scheduler.max_num_batched_tokens = 12
    try:
        outs = eng.generate(prompts, SamplingParams(temperature=1.0, max_tokens=9, top_k=1, ignore_eos=True))
        assert len(eng.scheduler.block_manager.free_block_ids) == 8 and eng.scheduler.state_slots.available() == 3
    finally:
        eng.exit()
    for p, o in zip(prompts, outs):
        gen = o["token_ids"]
        assert len(gen) == 9
        logits = O.forward(sd, cfg, p + gen)
        for k, t in enumerate(gen):
            row = logits[len(p) + k - 1]
            assert row[t] >= row.max() - 1e-4 * row.abs().max()


def test_checkpoint_loading_is_strict_and_the_registry_finds_the_design(tmp_path):
    import json
    from safetensors.torch import save_file
    from nano_qwen3tts_vllm_b200.config import RidevikConfig, load_model_config
    from nano_qwen3tts_vllm_b200.llm import LLM
    cfg = O.random_config(8, n_layers=3, share={2: 1})
    sd = {k: v.to(torch.bfloat16) for k, v in O.random_weights(cfg, seed=2).items()}
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    save_file(sd, str(tmp_path / "model.safetensors"))
    assert isinstance(load_model_config(str(tmp_path)), RidevikConfig)
    eng = LLM(str(tmp_path), dtype="float32", kvcache_block_size=16, num_kvcache_blocks=4, max_num_seqs=2, max_model_len=64,
              max_num_batched_tokens=128, enforce_eager=True)
    try:
        toks = tokens_for(cfg, 30, 1)
        assert nerr(replay(eng, {"a": toks}, [[("a", 30)]])["a"], O.forward(sd, cfg, toks)) < 2e-5
        model = eng.model_runner.model
        with pytest.raises(KeyError):
            model.load_state_dict({k: v for k, v in sd.items() if k != "l1.mix.sink"})
        with pytest.raises(KeyError):
            model.load_state_dict(dict(sd, **{"l2.shift": sd["l1.shift"]}))          # a sharing layer has no tensors
    finally:
        eng.exit()
