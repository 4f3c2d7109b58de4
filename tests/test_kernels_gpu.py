"""Native sm_100a kernels against plain PyTorch fp32 references of the same op (run on a B200)."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda"


def rel(a, b):
    a, b = a.float().cpu(), b.float().cpu()
    return ((a - b).abs().max() / (b.abs().max() + 1e-6)).item()


@pytest.fixture(scope="module")
def ops():
    from verl_b200.ops import native

    assert native.load(), "native library must load on a GPU box"
    return native.ops()


@pytest.mark.parametrize("shape", [(128, 256, 64), (300, 520, 200), (1000, 3584, 3584), (77, 152, 72), (320, 4608, 3584)])
@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, False), (True, True)])
def test_gemm_layouts(ops, shape, a_mn, b_mn):
    M, N, K = shape
    if a_mn and M % 8:
        pytest.skip("transposed A needs a 16-byte aligned row stride")
    torch.manual_seed(0)
    A = torch.randn(M, K, device=DEV).bfloat16()
    B = torch.randn(N, K, device=DEV).bfloat16()
    ref = A.float() @ B.float().t()
    a = A.t().contiguous() if a_mn else A
    b = B.t().contiguous() if b_mn else B
    d = ops.gemm(a, b, None, None, a_mn, b_mn, False, False, 0)
    torch.cuda.synchronize()
    assert int(ops.gemm_status()) == 0
    assert rel(d, ref) < 1e-2


def test_gemm_bias_fp32_accumulate(ops):
    torch.manual_seed(1)
    A = torch.randn(512, 384, device=DEV).bfloat16()
    B = torch.randn(1024, 384, device=DEV).bfloat16()
    bias = torch.randn(1024, device=DEV).bfloat16()
    d = ops.gemm(A, B, bias, None, False, False, False, False, 0)
    assert rel(d, A.float() @ B.float().t() + bias.float()) < 1e-2
    out = torch.randn(512, 1024, device=DEV)
    ref = out + A.float() @ B.float().t()
    ops.gemm(A, B, None, out, False, False, True, True, 0)
    assert rel(out, ref) < 1e-5


@pytest.mark.parametrize("shape", [(320, 3584, 18944), (320, 4608, 3584), (77, 264, 4096), (130, 1024, 8192)])
def test_gemm_k_split(ops, shape):
    """GEMMs with few output tiles and a deep K run K-split in the general kernel (the layouts the transposed kernel for
    few tokens does not serve: fp32 accumulation into the output, B stored [K, N]); partial sums are folded by the reduce
    launch or, with VERL_B200_SPLITK_FOLD=1, by the split that finishes a slab last. Several launches in a row: the slab
    counters return to zero by themselves."""
    M, N, K = shape
    assert int(ops.gemm_suggest_splits(M, N, K)) > 1
    torch.manual_seed(2)
    A = (torch.randn(M, K, device=DEV) * 0.5).bfloat16()
    B = (torch.randn(N, K, device=DEV) * 0.5).bfloat16()
    ref = A.float() @ B.float().t()
    Bt = B.t().contiguous()
    n0 = int(ops.launch_count())
    for _ in range(3):
        d2 = ops.gemm(A, Bt, None, None, False, True, False, False, 0)   # B stored [K, N]
        assert rel(d2, ref) < 1e-2
    assert int(ops.launch_count()) - n0 == (3 if int(ops.gemm_fold_in_kernel()) else 6)
    out = torch.randn(M, N, device=DEV)
    want = out + ref
    ops.gemm(A, B, None, out, False, False, True, True, 0)        # fp32 output, accumulate
    assert rel(out, want) < 1e-4
    assert int(ops.gemm_status()) == 0


@pytest.mark.parametrize("shape", [(320, 4608, 3584), (320, 3584, 18944), (320, 37888, 3584), (1, 256, 64), (5, 264, 72), (16, 128, 4096),
                                   (77, 152, 200), (130, 1024, 8192), (256, 3584, 3584), (257, 520, 1024), (512, 4608, 3584),
                                   (320, 2304, 3584), (64, 151936, 896), (640, 4608, 3584), (640, 3584, 1792), (1000, 264, 512)])
def test_gemm_few_tokens_transposed_kernel(ops, shape):
    """Up to 512 tokens per CTA (up to 1024 as two token blocks of the same launch): the kernel that puts 128 weight rows on the tensor core's M axis and all tokens on its N axis, K
    split over CTAs whose partial sums every split folds for its own share of the rows inside the same launch. Against
    the fp32 product, with bias, row-strided input and output, several launches in a row (the counters of a tile return
    to zero), and bit-equal across launches."""
    M, N, K = shape
    s = int(ops.gemm_skinny_splits(M, N, K))
    assert s >= 1
    torch.manual_seed(3)
    A = (torch.randn(M, K, device=DEV) * 0.5).bfloat16()
    B = (torch.randn(N, K, device=DEV) * 0.5).bfloat16()
    bias = torch.randn(N, device=DEV).bfloat16()
    ref = A.float() @ B.float().t() + bias.float()
    n0 = int(ops.launch_count())
    outs = [ops.gemm(A, B, bias, None, False, False, False, False, 0) for _ in range(3)]
    assert int(ops.launch_count()) - n0 == 3
    torch.cuda.synchronize()
    assert int(ops.gemm_status()) == 0
    assert rel(outs[0], ref) < 1e-2
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2])
    # a view into a wider buffer as input (row stride > K) and as output (row stride > N)
    wide = torch.zeros(M, K + 64, device=DEV, dtype=torch.bfloat16)
    wide[:, 8 : 8 + K] = A
    big = torch.full((M, N + 24), 7.0, device=DEV, dtype=torch.bfloat16)
    ops.gemm(wide[:, 8 : 8 + K], B, None, big[:, 8 : 8 + N], False, False, False, False, 0)
    assert rel(big[:, 8 : 8 + N], ref - bias.float()) < 1e-2
    assert bool((big[:, :8] == 7).all()) and bool((big[:, 8 + N :] == 7).all())
    assert int(ops.gemm_status()) == 0


@pytest.mark.parametrize("M", [320, 640, 37, 1000])
def test_gemm_row_ranges_of_a_fused_weight(ops, M):
    """The q | k | v rows of one tensor-parallel rank inside the replicated fused projection weight (and gate | up; ranges
    that are no multiple of 128 rows) as one launch: outputs side by side, bias taken by weight row."""
    from verl_b200.ops import functional as F

    torch.manual_seed(5)
    K = 3584
    for total, ranges in ((4608, [(1792, 1792), (3584 + 256, 256), (4096 + 256, 256)]), (2 * 1184, [(0, 592), (1184, 592)]),
                          (1024, [(8, 200), (512, 72), (600, 128), (900, 24)])):
        A = (torch.randn(M, K, device=DEV) * 0.5).bfloat16()
        Wt = (torch.randn(total, K, device=DEV) * 0.5).bfloat16()
        bias = torch.randn(total, device=DEV).bfloat16()
        n0 = int(ops.launch_count())
        out = F.gemm_row_ranges(A, Wt, bias, ranges)
        assert int(ops.launch_count()) - n0 == 1
        ref = torch.cat([A.float() @ Wt[w0 : w0 + r].float().t() + bias[w0 : w0 + r].float() for w0, r in ranges], dim=1)
        assert out.shape == ref.shape and rel(out, ref) < 1e-2
        out2 = F.gemm_row_ranges(A, Wt, None, ranges)
        assert rel(out2, ref - torch.cat([bias[w0 : w0 + r].float() for w0, r in ranges]).unsqueeze(0)) < 1e-2
    torch.cuda.synchronize()
    assert int(ops.gemm_status()) == 0


@pytest.mark.parametrize("shape", [(300, 520, 200), (2048, 1184, 512), (1500, 4736, 3584), (128, 64, 64)])
def test_gemm_with_swiglu_epilogue(ops, shape):
    """Up-projection of a gated MLP with the activation in the GEMM epilogue: the stacked [gate; up] weight is read through
    a 3-D tensor map that interleaves the halves row by row, so that a thread holds both members of every pair. Against
    the fp32 product; the pre-activation output has the stacked layout of the separate GEMM."""
    M, I, K = shape
    torch.manual_seed(4)
    A = (torch.randn(M, K, device=DEV) * 0.5).bfloat16()
    Wt = (torch.randn(2 * I, K, device=DEV) * 0.1).bfloat16()
    gu_ref = A.float() @ Wt.float().t()
    act_ref = torch.nn.functional.silu(gu_ref[:, :I]) * gu_ref[:, I:]
    act, gu = ops.gemm_swiglu(A, Wt, True)
    torch.cuda.synchronize()
    assert int(ops.gemm_status()) == 0
    assert act.shape == (M, I) and gu.shape == (M, 2 * I)
    assert rel(gu, gu_ref) < 1e-2 and rel(act, act_ref) < 1e-2
    act2, none = ops.gemm_swiglu(A, Wt, False)
    assert none.numel() == 0 and torch.equal(act, act2)
    # the separate kernels on the same inputs agree up to the bf16 rounding of the pre-activation
    sep = ops.swiglu_fwd(ops.gemm(A, Wt, None, None, False, False, False, False, 0))
    assert rel(act, sep) < 2e-2


def test_rmsnorm_fwd_bwd(ops):
    from verl_b200.ops import functional as F

    torch.manual_seed(0)
    T, H = 1000, 3584
    x, r = torch.randn(T, H).bfloat16(), torch.randn(T, H).bfloat16()
    w = (torch.rand(H) + 0.5).bfloat16()
    y, xe, rs = F.rms_norm(x.to(DEV), w.to(DEV), 1e-6, r.to(DEV))
    y2, xe2, rs2 = F.rms_norm(x.float(), w.float(), 1e-6, r.float())
    assert rel(y, y2) < 1e-2 and rel(xe, xe2) < 1e-2 and rel(rs, rs2) < 1e-3
    dy, dres = torch.randn(T, H).bfloat16(), torch.randn(T, H).bfloat16()
    dw, dw2 = torch.zeros(H, device=DEV), torch.zeros(H)
    dx = F.rms_norm_bwd(dy.to(DEV), xe.to(DEV), w.to(DEV), rs, dres.to(DEV), dw, True)
    dx2 = F.rms_norm_bwd(dy.float(), xe.float().cpu(), w.float(), rs.cpu(), dres.float(), dw2, True)
    assert rel(dx, dx2) < 1e-2 and rel(dw, dw2) < 1e-4


def test_rope_swiglu_embedding(ops):
    from verl_b200.ops import functional as F

    torch.manual_seed(0)
    T = 777
    q = torch.randn(T, 28, 128).bfloat16()
    pos = torch.randint(0, 4000, (T,), dtype=torch.int32)
    c, s = F.rope_table(4096, 128, 1e6, "cpu")
    a = F.apply_rope_(q.clone().to(DEV), pos.to(DEV), c.to(DEV), s.to(DEV))
    assert rel(a, F.apply_rope_(q.float().clone(), pos, c, s)) < 1e-2
    back = F.apply_rope_(a.clone(), pos.to(DEV), c.to(DEV), s.to(DEV), backward=True)
    assert rel(back, q) < 1e-2
    gu, do = torch.randn(T, 2 * 4864).bfloat16(), torch.randn(T, 4864).bfloat16()
    assert rel(F.swiglu(gu.to(DEV)), F.swiglu(gu.float())) < 1e-2
    assert rel(F.swiglu_bwd(do.to(DEV), gu.to(DEV)), F.swiglu_bwd(do.float(), gu.float())) < 1e-2
    W, ids = torch.randn(5000, 896).bfloat16(), torch.randint(0, 5000, (T,))
    assert rel(F.embedding(ids.to(DEV), W.to(DEV)), F.embedding(ids, W.float())) == 0
    dW, dW2 = torch.zeros(5000, 896, device=DEV), torch.zeros(5000, 896)
    dy = torch.randn(T, 896).bfloat16()
    F.embedding_bwd_(ids.to(DEV), dy.to(DEV), dW)
    F.embedding_bwd_(ids, dy.float(), dW2)
    assert rel(dW, dW2) < 1e-5


def test_fused_lm_head_forward_backward(ops):
    from verl_b200.ops import functional as F

    torch.manual_seed(0)
    T, H, V = 700, 896, 151936
    h = (torch.randn(T, H) * 0.5).bfloat16()
    W = (torch.randn(V, H) * 0.05).bfloat16()
    lab = torch.randint(0, V, (T,))
    lp, ent, lse = F.lmhead_logprob_entropy(h.to(DEV), W.to(DEV), lab.to(DEV), 0.8)
    lp2, ent2, lse2 = F.lmhead_logprob_entropy(h.float(), W.float(), lab, 0.8)
    assert (lp.cpu() - lp2).abs().max() < 2e-3 and (ent.cpu() - ent2).abs().max() < 2e-3 and (lse.cpu() - lse2).abs().max() < 2e-3
    glp, gent = torch.randn(T), torch.randn(T) * 0.1
    dW = torch.zeros(V, H, device=DEV)
    dh = F.lmhead_backward(h.to(DEV), W.to(DEV), lab.to(DEV), 0.8, lse, ent, glp.to(DEV), gent.to(DEV), dW)
    dW2 = torch.zeros(V, H)
    dh2 = F.lmhead_backward(h.float(), W.float(), lab, 0.8, lse2, ent2, glp, gent, dW2)
    assert rel(dh, dh2) < 2e-2 and rel(dW, dW2) < 2e-2
    assert int(ops.gemm_status()) == 0


def test_adamw_matches_torch(ops):
    torch.manual_seed(0)
    n = 100003
    p, g = torch.randn(n), torch.randn(n)
    pp = torch.nn.Parameter(p.clone())
    opt = torch.optim.AdamW([pp], lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.01)
    ctrl = torch.zeros(4, device=DEV)
    pd, gd, md, vd = p.to(DEV), g.to(DEV), torch.zeros(n, device=DEV), torch.zeros(n, device=DEV)
    ob = torch.empty(n, device=DEV, dtype=torch.bfloat16)
    for step in range(1, 4):
        pp.grad = g.clone()
        torch.nn.utils.clip_grad_norm_([pp], 1.0)
        opt.step()
        ctrl.zero_()
        ops.sumsq_(gd, ctrl)
        ops.clip_coef_(ctrl, 1.0)
        ops.adamw_(pd, gd, md, vd, ob, ctrl, 1e-3, 0.9, 0.999, 1e-8, 0.01, step, 1.0, False)
    assert rel(pd, pp.data) < 1e-5 and abs(ctrl[3].item() - g.norm().item()) < 1e-2
    assert rel(ob, pp.data) < 1e-2
    # a non-finite gradient skips the update
    gd[0] = float("inf")
    before = pd.clone()
    ctrl.zero_()
    ops.sumsq_(gd, ctrl)
    ops.clip_coef_(ctrl, 1.0)
    ops.adamw_(pd, gd, md, vd, ob, ctrl, 1e-3, 0.9, 0.999, 1e-8, 0.01, 4, 1.0, False)
    assert torch.equal(pd, before) and ctrl[2].item() == 1.0


def test_paged_decode_attention_and_kv_append(ops):
    from verl_b200.ops import functional as F

    torch.manual_seed(0)
    B, nh, nkv, hd, bs, nb = 5, 28, 4, 128, 16, 64
    kc, vc = torch.randn(nb, bs, nkv, hd).bfloat16(), torch.randn(nb, bs, nkv, hd).bfloat16()
    bt = torch.stack([torch.randperm(nb)[:12] for _ in range(B)]).to(torch.int32)
    cl = torch.tensor([1, 17, 100, 190, 64], dtype=torch.int32)
    q = torch.randn(B, nh, hd).bfloat16()
    o = F.paged_decode_attention(q.to(DEV), kc.to(DEV), vc.to(DEV), bt.to(DEV), cl.to(DEV))
    assert rel(o, F.paged_decode_attention(q.float(), kc.float(), vc.float(), bt, cl)) < 1e-2
    kd, vd = torch.zeros(nb, bs, nkv, hd, device=DEV, dtype=torch.bfloat16), torch.zeros(nb, bs, nkv, hd, device=DEV, dtype=torch.bfloat16)
    k, v = torch.randn(7, nkv, hd).bfloat16(), torch.randn(7, nkv, hd).bfloat16()
    slots = torch.tensor([3, 900, -1, 5, 77, 1023, 0])
    F.kv_append_(k.to(DEV), v.to(DEV), slots.to(DEV), kd, vd)
    flat = kd.view(-1, nkv, hd).cpu()
    assert torch.equal(flat[900], k[1]) and torch.equal(flat[0], k[6]) and flat[1].abs().sum() == 0


@pytest.mark.parametrize("nh,nkv,hd", [(28, 4, 128), (14, 2, 64)])
def test_grouped_prefix_paged_decode_matches_reference(ops, nh, nkv, hd):
    """Sequences that share their leading pages in groups: the group kernel + per-sequence kernel + merge give the fp32
    reference; members of different sizes, a sequence in no group, an inactive member, an empty group row, and a group
    whose shared pages do not divide evenly over the prefix splits."""
    from verl_b200.ops import functional as F

    torch.manual_seed(3)
    B, bs, nb, maxb = 12, 64, 96, 10
    kc, vc = torch.randn(nb, bs, nkv, hd).bfloat16(), torch.randn(nb, bs, nkv, hd).bfloat16()
    perm = torch.randperm(nb).tolist()
    bt = torch.zeros(B, maxb, dtype=torch.int32)
    take = lambda n: [perm.pop() for _ in range(n)]
    groups = {0: ([0, 1, 2, 3, 4], 3), 1: ([5, 6], 5), 3: ([7, 8, 9], 1)}     # gid -> (member sequences, shared pages); gid 2 stays empty
    cl = torch.zeros(B, dtype=torch.int32)
    skip = torch.zeros(B, dtype=torch.int32)
    for gid, (members, pages) in groups.items():
        shared = take(pages)
        for j, b in enumerate(members):
            own = take(3)
            bt[b, :pages] = torch.tensor(shared, dtype=torch.int32)
            bt[b, pages:pages + 3] = torch.tensor(own, dtype=torch.int32)
            cl[b] = pages * bs + 1 + 37 * j + (bs if j == 1 else 0)              # ragged tails, some reaching a second own page
            skip[b] = pages
    for b in (10, 11):                                                           # in no group
        bt[b, :4] = torch.tensor(take(4), dtype=torch.int32)
        cl[b] = 70 + 100 * (b - 10)
    cl[8] = 0                                                                    # an inactive member of group 3
    members = torch.full((4, 8), -1, dtype=torch.int32)
    grp_pages = torch.zeros(4, dtype=torch.int32)
    for gid, (m, pages) in groups.items():
        members[gid, : len(m)] = torch.tensor(m, dtype=torch.int32)
        grp_pages[gid] = pages
    q = torch.randn(B, nh, hd).bfloat16()
    ref = F.paged_decode_attention(q.float(), kc.float(), vc.float(), bt, cl)
    for psplit, nsplit in ((2, 1), (1, 2), (3, 3)):
        ws = torch.empty(B * nh * (psplit + nsplit) * (hd + 2), device=DEV)
        ws.fill_(float("nan"))                                                   # stale scratch must not leak into the result
        o = F.paged_decode_attention(q.to(DEV), kc.to(DEV), vc.to(DEV), bt.to(DEV), cl.to(DEV),
                                     groups=(members.to(DEV), grp_pages.to(DEV), skip.to(DEV), ws, psplit, nsplit))
        torch.cuda.synchronize()
        live = cl > 0
        assert torch.isfinite(o[live.to(DEV)]).all()
        assert rel(o[live.to(DEV)], ref[live]) < 1e-2, (psplit, nsplit, rel(o[live.to(DEV)], ref[live]))
        plain = F.paged_decode_attention(q.to(DEV), kc.to(DEV), vc.to(DEV), bt.to(DEV), cl.to(DEV))
        assert rel(o[live.to(DEV)], plain[live.to(DEV)]) < 5e-3
    assert int(ops.gemm_status()) == 0


@pytest.mark.parametrize("nh,nkv,hd", [(28, 4, 128), (14, 2, 64)])
def test_fused_rope_kv_append_matches_the_separate_ops(ops, nh, nkv, hd):
    from verl_b200.ops import functional as F

    torch.manual_seed(5)
    T, nb, bs = 37, 8, 64
    qkv = torch.randn(T, (nh + 2 * nkv) * hd).bfloat16().to(DEV)
    pos = torch.randint(0, 500, (T,), dtype=torch.int32, device=DEV)
    inv = 1.0 / (1e4 ** (torch.arange(0, hd, 2).float() / hd))
    ang = torch.arange(512).float()[:, None] * inv[None]
    cos, sin = ang.cos().to(DEV), ang.sin().to(DEV)
    slots = torch.randperm(nb * bs)[:T].to(DEV)
    slots[3] = -1                                                     # an inactive sequence: q is rotated, nothing is appended
    kc, vc = (torch.zeros(nb, bs, nkv, hd, dtype=torch.bfloat16, device=DEV) for _ in range(2))
    fused = qkv.clone()
    F.rope_kv_append_(fused, pos, cos, sin, slots, kc, vc, nh, nkv, hd)
    ref = qkv.clone()
    q = ref[:, : nh * hd].view(T, nh, hd)
    k = ref[:, nh * hd : (nh + nkv) * hd].view(T, nkv, hd)
    v = ref[:, (nh + nkv) * hd :].view(T, nkv, hd)
    kc2, vc2 = torch.zeros_like(kc), torch.zeros_like(vc)
    F.apply_rope_(q, pos, cos, sin)
    F.apply_rope_(k, pos, cos, sin)
    F.kv_append_(k, v, slots, kc2, vc2)
    torch.cuda.synchronize()
    assert torch.equal(fused, ref) and torch.equal(kc, kc2) and torch.equal(vc, vc2)
    # and against fp32 math on the host
    half = hd // 2
    x = qkv.float().cpu()[:, : nh * hd].view(T, nh, hd)
    c, s_ = cos.cpu()[pos.cpu().long()][:, None], sin.cpu()[pos.cpu().long()][:, None]
    want = torch.cat([x[..., :half] * c - x[..., half:] * s_, x[..., half:] * c + x[..., :half] * s_], -1)
    assert rel(fused[:, : nh * hd].view(T, nh, hd), want) < 1e-2


def _attn_reference(q, k, v, lens, scale):
    """fp32 causal GQA attention per sequence with autograd."""
    outs, off = [], 0
    G = q.shape[1] // k.shape[1]
    for n in lens:
        qs, ks, vs = (t[off:off + n].float() for t in (q, k, v))
        ks, vs = ks.repeat_interleave(G, 1), vs.repeat_interleave(G, 1)
        s = torch.einsum("qhd,khd->hqk", qs, ks) * scale
        s = s.masked_fill(torch.triu(torch.ones(n, n, dtype=torch.bool, device=q.device), 1), float("-inf"))
        outs.append(torch.einsum("hqk,khd->qhd", torch.softmax(s, -1), vs))
        off += n
    return torch.cat(outs, 0)


@pytest.mark.parametrize("lens,nh,nkv", [([300, 129, 64, 1], 4, 2), ([1000], 7, 1), ([130, 257], 2, 2),
                                         ([3072, 2900], 28, 4)])   # the last: the benchmark's shape class (long rows, 28 / 4 heads)
def test_attention_forward_and_backward_tcgen05(ops, lens, nh, nkv):
    torch.manual_seed(0)
    T, hd = sum(lens), 128
    scale = 1.0 / math.sqrt(hd)
    q = (torch.randn(T, nh, hd, device=DEV) * 0.7).bfloat16()
    k = (torch.randn(T, nkv, hd, device=DEV) * 0.7).bfloat16()
    v = torch.randn(T, nkv, hd, device=DEV).bfloat16()
    do = torch.randn(T, nh, hd, device=DEV).bfloat16()
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32, device=DEV)
    out, lse = ops.attn_fwd(q, k, v, cu, scale)
    qr, kr, vr = (t.detach().float().requires_grad_(True) for t in (q, k, v))
    ref = _attn_reference(qr, kr, vr, lens, scale)
    assert rel(out, ref) < 2e-2
    dq_r, dk_r, dv_r = torch.autograd.grad(ref, (qr, kr, vr), do.float())
    dq, dk, dv = ops.attn_bwd(do, q, k, v, out, lse, cu, max(lens), scale)
    assert ops.gemm_status() == 0
    assert rel(dv, dv_r) < 3e-2 and rel(dk, dk_r) < 3e-2 and rel(dq, dq_r) < 3e-2, (rel(dq, dq_r), rel(dk, dk_r), rel(dv, dv_r))


def test_moe_router_grouped_gemm_and_layer_match_reference(ops, monkeypatch):
    from verl_b200.models import DecoderModel, FlatParams
    from verl_b200.models.config import ModelConfig

    torch.manual_seed(0)
    # router kernel against softmax + topk
    logits = torch.randn(700, 64, device=DEV).bfloat16()
    w, idx, counts = ops.moe_route_topk(logits, 4, True)
    pr = torch.softmax(logits.float(), -1)
    rw, ri = torch.topk(pr, 4, -1)
    rw = rw / rw.sum(-1, keepdim=True)
    assert torch.equal(idx.long().sort(-1).values, ri.sort(-1).values) and rel(w.sort(-1).values, rw.sort(-1).values) < 1e-4
    assert torch.equal(counts.long(), torch.bincount(ri.reshape(-1), minlength=64))
    # one MoE layer: native (grouped tcgen05 GEMMs) against the per-expert fallback, forward and all gradients
    cfg = ModelConfig(model_type="qwen3_moe", vocab_size=512, hidden_size=256, intermediate_size=256, num_hidden_layers=1,
                      num_attention_heads=4, num_key_value_heads=2, head_dim=64, num_experts=32, num_experts_per_tok=4,
                      moe_intermediate_size=128, eos_token_id=2, pad_token_id=0)
    outs = {}
    for native_on in ("1", "0"):
        monkeypatch.setenv("VERL_B200_MOE_NATIVE", native_on)
        P = FlatParams(cfg, dtype=torch.bfloat16, device=DEV, with_main_grad=True)
        P.init_weights(seed=4, std=0.05)
        model = DecoderModel(cfg, P)
        W = P.layer(0)
        h2 = (torch.randn(700, 256, device=DEV, generator=torch.Generator(device=DEV).manual_seed(1))).bfloat16()
        g = (torch.randn(700, 256, device=DEV, generator=torch.Generator(device=DEV).manual_seed(2))).bfloat16()
        S = {}
        out = model._moe_fwd(W, h2, S)
        gh = model._moe_bwd(W, g, h2, S)
        outs[native_on] = (out, gh, W["mlp.experts.gate_up_proj"].main_grad.clone(), W["mlp.experts.down_proj"].main_grad.clone(),
                           W["mlp.gate.weight"].main_grad.clone())
    assert ops.gemm_status() == 0
    for a, b in zip(outs["1"], outs["0"]):
        assert rel(a, b) < 3e-2, rel(a, b)


@pytest.mark.parametrize("shape", [(320, 4608, 3584), (77, 136, 256), (1000, 1024, 1024)])
def test_fp8_block_scaled_quant_and_gemm(ops, shape):
    from verl_b200.ops import functional as F

    torch.manual_seed(0)
    M, N, K = shape
    x = torch.randn(M, K, device=DEV).bfloat16()
    w = (torch.randn(N, K, device=DEV) * 0.05).bfloat16()
    xq, xs = F.fp8_quantize_1x128(x)
    xq_c, xs_c = F.fp8_quantize_1x128(x.cpu())
    assert rel(xs, xs_c) < 1e-6 and (xq.cpu() != xq_c).float().mean() < 1e-2  # identical up to rounding ties (reciprocal multiply vs division)
    assert rel(F.fp8_dequantize_1x128(xq.cpu(), xs.cpu()), x.float()) < 0.07
    wq, ws = F.fp8_quantize_1x128(w)
    y = F.linear_fp8(x, wq, ws)
    ref = F.fp8_dequantize_1x128(xq.cpu(), xs.cpu()) @ F.fp8_dequantize_1x128(wq.cpu(), ws.cpu()).t()
    assert ops.gemm_status() == 0
    assert rel(y, ref) < 1e-2  # same quantised operands: only accumulation order and the bf16 output rounding differ
    assert rel(y, x.float().cpu() @ w.float().cpu().t()) < 0.06  # against the unquantised product


def test_sampler_distribution_and_logprob(ops):
    from verl_b200.ops import functional as F

    torch.manual_seed(0)
    V = 152064
    lg = (torch.randn(4, V) * 2).bfloat16()
    tok, lp = F.sample_tokens(lg.to(DEV), 1.0, torch.arange(4).to(DEV), 3, valid_vocab=V)
    ref = torch.log_softmax(lg.float(), -1).gather(-1, tok.cpu().unsqueeze(-1)).squeeze(-1)
    assert (lp.cpu() - ref).abs().max() < 1e-3
    tok, _ = F.sample_tokens(lg.to(DEV), 0.0, torch.arange(4).to(DEV), 3, valid_vocab=V)
    assert torch.equal(tok.cpu(), lg.float().argmax(-1))
    lg2 = torch.tensor([[0.0, 1.0, 2.0, 3.0] + [-30.0] * 60]).bfloat16().repeat(4000, 1)
    tok, _ = F.sample_tokens(lg2.to(DEV), 1.0, torch.arange(4000).to(DEV), 0)
    hist = torch.bincount(tok.cpu(), minlength=4)[:4].float() / 4000
    assert (hist - torch.softmax(torch.tensor([0.0, 1, 2, 3]), 0)).abs().max() < 0.03
    # vocabulary masking
    tok, _ = F.sample_tokens(lg.to(DEV), 1.0, torch.arange(4).to(DEV), 5, valid_vocab=100)
    assert int(tok.max()) < 100


def _kept_set(x: torch.Tensor, temperature: float, top_k: int, top_p: float) -> torch.Tensor:
    """Reference of the filtered sampler's kept set for one row (fp64): the k largest values and whatever ties with the
    k-th, then the smallest set of largest values whose mass reaches top_p of that, ties with the boundary value kept."""
    x = x.double() / temperature
    keep = torch.ones_like(x, dtype=torch.bool)
    if 0 < top_k < x.numel():
        keep &= x >= torch.topk(x, top_k).values[-1]
    if top_p < 1.0:
        e = torch.where(keep, torch.exp(x - x.max()), torch.zeros_like(x))
        vals, inv = torch.unique(x, return_inverse=True)           # ascending
        group = torch.zeros_like(vals).index_add_(0, inv, e)
        cum_from_top = torch.flip(torch.cumsum(torch.flip(group, [0]), 0), [0])
        # the boundary group is the highest-valued group (scanning down) at which the cumulative mass reaches the target
        reached = cum_from_top >= top_p * e.sum()
        boundary = vals[reached.nonzero().max()]
        keep &= x >= boundary
    return keep


def test_filtered_sampler_top_k_top_p(ops):
    from verl_b200.ops import functional as F

    torch.manual_seed(1)
    # (a) full vocabulary, ties everywhere (bf16 logits): token inside the kept set, log-prob of the renormalised distribution
    V, B = 152064, 6
    lg = (torch.randn(B, V) * 2.5).bfloat16()
    for temperature, top_k, top_p in ((1.0, 50, 1.0), (0.7, -1, 0.9), (1.3, 200, 0.5), (1.0, 1, 1.0), (1.0, -1, 0.01)):
        tok, lp = F.sample_tokens(lg.to(DEV), temperature, torch.arange(B).to(DEV) + 7, 11, valid_vocab=V, top_k=top_k, top_p=top_p)
        tok, lp = tok.cpu(), lp.cpu()
        for r in range(B):
            keep = _kept_set(lg[r].float(), temperature, top_k, top_p)
            assert bool(keep[tok[r]]), (temperature, top_k, top_p, r)
            xs = lg[r].double() / temperature
            ref = xs[tok[r]] - torch.logsumexp(xs[keep], 0)
            assert abs(float(lp[r]) - float(ref)) < 2e-3, (temperature, top_k, top_p, r, float(lp[r]), float(ref))
        if top_k == 1:  # the maximum (any of its ties)
            assert torch.equal(lg.float().gather(1, tok.unsqueeze(1)).squeeze(1), lg.float().max(-1).values)
    # (b) empirical distribution on a small row of distinct values: top-k = 3 keeps {3, 2, 1}, top-p = 0.6 keeps {3} u {2}
    row = torch.tensor([[0.0, 1.0, 2.0, 3.0] + [-30.0] * 60]).bfloat16().repeat(6000, 1).to(DEV)
    tok, _ = F.sample_tokens(row, 1.0, torch.arange(6000).to(DEV), 0, top_k=3)
    hist = torch.bincount(tok.cpu(), minlength=4)[:4].float() / 6000
    want = torch.softmax(torch.tensor([1.0, 2.0, 3.0]), 0)
    assert hist[0] == 0 and (hist[1:] - want).abs().max() < 0.03
    tok, _ = F.sample_tokens(row, 1.0, torch.arange(6000).to(DEV), 0, top_p=0.7)   # p(3) = 0.64 < 0.7 <= p(3) + p(2)
    hist = torch.bincount(tok.cpu(), minlength=4)[:4].float() / 6000
    assert hist[0] == 0 and hist[1] == 0 and (hist[2:] - torch.softmax(torch.tensor([2.0, 3.0]), 0)).abs().max() < 0.03
    # (c) vocabulary mask and negative logits only
    neg = (-torch.rand(3, 5000) * 20 - 1).bfloat16()
    tok, lp = F.sample_tokens(neg.to(DEV), 1.0, torch.arange(3).to(DEV), 2, valid_vocab=1000, top_k=5, top_p=0.95)
    for r in range(3):
        keep = _kept_set(neg[r, :1000].float(), 1.0, 5, 0.95)
        assert int(tok[r]) < 1000 and bool(keep[int(tok[r])])


def test_advantage_kernels(ops):
    import numpy as np

    from verl_b200.ops import functional as F
    from verl_b200.trainer.ppo import core_algos as ca

    torch.manual_seed(0)
    B, L = 64, 200
    mask = (torch.rand(B, L) > 0.2).float()
    r = torch.zeros(B, L)
    r[:, -1] = torch.rand(B)
    g = torch.arange(B) // 8
    adv, scores = F.grpo_advantage(r.to(DEV), mask.to(DEV), g.to(DEV), 8)
    ref, _ = ca.compute_grpo_outcome_advantage(r, mask, np.array(g.tolist()))
    assert (adv.cpu() - ref).abs().max() < 1e-4
    v = torch.randn(B, L)
    rr = torch.randn(B, L) * 0.1
    a, ret = F.gae_advantage(rr.to(DEV), v.to(DEV), mask.to(DEV), 0.99, 0.95, True)
    a2, ret2 = ca.compute_gae_advantage_return(rr, v, mask, 0.99, 0.95)
    assert (ret.cpu() - ret2).abs().max() < 1e-4 and (a.cpu() - a2).abs().max() < 1e-3


@pytest.mark.parametrize("name", ["tiny-qwen2", "tiny-llama", "tiny-moe", "tiny-qwen2-moe"])
def test_model_gpu_matches_cpu(ops, name):
    from verl_b200.models import DecoderModel, FlatParams, PackedBatch, get_preset

    torch.manual_seed(0)
    cfg = get_preset(name)
    P = FlatParams(cfg, dtype=torch.float32, with_main_grad=True)
    P.init_weights(seed=1, std=0.05)
    Pg = FlatParams(cfg, dtype=torch.bfloat16, device=DEV, with_main_grad=True)
    Pg.flat.copy_(P.flat)
    P.flat.copy_(Pg.flat.float().cpu())
    lengths = [37, 64, 128, 9]
    T = sum(lengths)
    ids, labels, w = torch.randint(3, cfg.vocab_size, (T,)), torch.randint(3, cfg.vocab_size, (T,)), torch.randn(T)
    for rec in ["none", "full"]:
        P.zero_grad()
        Pg.zero_grad()
        lp, ent = DecoderModel(cfg, P, recompute=rec).forward_logprobs(PackedBatch.from_lengths(ids, lengths), labels, 1.0)
        (lp * w).sum().backward()
        lpg, entg = DecoderModel(cfg, Pg, recompute=rec).forward_logprobs(PackedBatch.from_lengths(ids, lengths, device=DEV), labels.to(DEV), 1.0)
        (lpg * w.to(DEV)).sum().backward()
        if cfg.is_moe:
            # bf16 router logits flip the expert choice of tokens that sit on a near-tie: most tokens agree closely, a few differ
            assert ((lpg.cpu() - lp).abs() < 0.05).float().mean() > 0.9 and ((entg.cpu() - ent).abs() < 0.02).float().mean() > 0.9
            assert rel(Pg.main_grad, P.main_grad) < 0.35
        else:
            assert (lpg.cpu() - lp).abs().max() < 0.05 and (entg.cpu() - ent).abs().max() < 0.02
            assert rel(Pg.main_grad, P.main_grad) < 0.05


def test_activation_offload_gives_identical_gradients(ops):
    from verl_b200.models import DecoderModel, FlatParams, PackedBatch, get_preset
    from verl_b200.utils.activation_offload import ActivationOffloader

    cfg = get_preset("tiny-llama")
    grads = []
    for use in (False, True):
        P = FlatParams(cfg, dtype=torch.bfloat16, device=DEV, with_main_grad=True)
        P.init_weights(seed=1, std=0.05)
        model = DecoderModel(cfg, P, recompute="full")
        if use:
            model.offloader = ActivationOffloader(DEV)
        g = torch.Generator().manual_seed(0)
        ids = torch.randint(3, cfg.vocab_size, (300,), generator=g).to(DEV)
        labels = torch.randint(3, cfg.vocab_size, (300,), generator=g).to(DEV)
        lp, ent = model.forward_logprobs(PackedBatch.from_lengths(ids, [120, 100, 80], device=DEV), labels, 1.0)
        (-lp.sum()).backward()
        torch.cuda.synchronize()
        grads.append(P.main_grad.clone())
        if use:
            assert model.offloader.bytes_offloaded > 0
    assert torch.equal(grads[0], grads[1])


def test_bounded_wait_runs_out_reports_status_and_gates_the_update(ops):
    """A barrier on a flag that nobody sets gives up after its limit: the status word says so, the device stays usable,
    and the poisoned norm accumulator makes the fused AdamW kernel skip (state untouched, old weights republished)."""
    import time

    assert int(ops.gemm_status()) == 0 and int(ops.comm_status()) == 0
    pads = [torch.zeros(64, dtype=torch.int32, device=DEV) for _ in range(2)]  # this GPU plays rank 0 of 2; "rank 1" never arrives
    ptrs = torch.tensor([p.data_ptr() for p in pads], dtype=torch.int64)
    ctrl = torch.zeros(4, device=DEV)
    torch.cuda.synchronize()
    t0 = time.time()
    ops.peer_barrier(ptrs, 0, 1, 0.2, ctrl[:1])
    torch.cuda.synchronize()
    assert 0.15 < time.time() - t0 < 5.0
    assert int(pads[0][0]) == 1 and int(pads[1][0]) == 1 and int(pads[0][1]) == 0  # own arrival was published to both pads
    assert torch.isinf(ctrl[0])
    assert int(ops.comm_status()) == 4 and int(ops.comm_status()) == 0  # reported once, then cleared
    # the step that follows: the sum of squares stays non-finite, the clip kernel raises the skip flag, AdamW leaves state alone
    n = 4096
    g = torch.randn(n, device=DEV)
    ops.sumsq_(g, ctrl)
    ops.clip_coef_(ctrl, 1.0)
    assert float(ctrl[2]) == 1.0
    master = torch.randn(n, device=DEV)
    m, v = torch.rand(n, device=DEV), torch.rand(n, device=DEV)
    m0, v0, master0 = m.clone(), v.clone(), master.clone()
    work = torch.zeros(n, dtype=torch.bfloat16, device=DEV)
    ops.adamw_allgather_(master, g, m, v, torch.tensor([work.data_ptr()], dtype=torch.int64), 0, 0, 0, ctrl, 1e-3, 0.9, 0.999, 1e-8, 0.01, 1)
    torch.cuda.synchronize()
    assert torch.equal(master, master0) and torch.equal(m, m0) and torch.equal(v, v0)
    assert torch.equal(work, master0.bfloat16())
    # a barrier whose peers have all arrived returns at once and poisons nothing
    pads[0][1] = 2
    ctrl.zero_()
    ops.peer_barrier(ptrs, 0, 2, 0.2, ctrl[:1])
    torch.cuda.synchronize()
    assert float(ctrl[0]) == 0.0 and int(ops.comm_status()) == 0
    assert float(torch.ones(8, device=DEV).sum()) == 8.0


def test_rollout_engine_cuda_graph_matches_eager(ops):
    from verl_b200.models import FlatParams, ModelConfig
    from verl_b200.workers.rollout.native.engine import RolloutEngine, SamplingParams

    cfg = ModelConfig(model_type="qwen2", vocab_size=2048, hidden_size=512, intermediate_size=1024, num_hidden_layers=2,
                      num_attention_heads=4, num_key_value_heads=2, head_dim=128, eos_token_id=-1, pad_token_id=0)
    P = FlatParams(cfg, dtype=torch.bfloat16, device=DEV)
    P.init_weights(seed=0, std=0.05)
    prompts = [[5, 6, 7, 8, 9], [10, 11, 12], [20, 21, 22, 23, 24, 25, 26], [3, 4], [7, 7, 7, 7]]
    outs = {}
    for graph in (True, False):
        eng = RolloutEngine(cfg, P, max_num_seqs=3, max_model_len=64, block_size=16, num_blocks=32, sync_interval=3,
                            use_cuda_graph=graph, eos_token_id=-1)
        outs[graph] = [o.token_ids for o in eng.generate(prompts, SamplingParams(temperature=0.0, max_tokens=9))]
    assert outs[True] == outs[False] and all(len(t) == 9 for t in outs[True])


def test_rollout_engine_grouped_decode_follows_its_groups(ops, monkeypatch):
    """The samples of a prompt decode as a group (shared prompt pages read once by the group kernel); groups shrink and
    dissolve as members finish at different lengths. Same log-probs as the per-sequence kernel, and the token sequences
    agree except where bf16 attention outputs tip a near-tie."""
    from verl_b200.models import FlatParams, ModelConfig
    from verl_b200.workers.rollout.native.engine import RolloutEngine, SamplingParams

    cfg = ModelConfig(model_type="qwen2", vocab_size=2048, hidden_size=512, intermediate_size=1024, num_hidden_layers=2,
                      num_attention_heads=4, num_key_value_heads=2, head_dim=128, eos_token_id=-1, pad_token_id=0)
    P = FlatParams(cfg, dtype=torch.bfloat16, device=DEV)
    P.init_weights(seed=0, std=0.05)
    g = torch.Generator().manual_seed(0)
    base = [torch.randint(3, 2048, (n,), generator=g).tolist() for n in (150, 70, 200)]   # 2, 1 and 3 full pages of 64
    prompts, params = [], []
    for i, p in enumerate(base):
        for j in range(4):                                                               # 4 samples per prompt, unequal lengths
            prompts.append(p)
            params.append(SamplingParams(temperature=1.0, max_tokens=6 + 5 * j + i, seed=100 * i + j, logprobs=True))
    prompts.append([9, 8, 7])                                                            # a request of its own
    params.append(SamplingParams(temperature=1.0, max_tokens=12, seed=999, logprobs=True))
    outs = {}
    for flag in ("1", "0"):
        monkeypatch.setenv("VERL_B200_GROUPED_DECODE", flag)
        eng = RolloutEngine(cfg, P, max_num_seqs=16, max_model_len=320, block_size=64, num_blocks=80, sync_interval=4, eos_token_id=-1)
        assert eng.grouped_decode == (flag == "1")
        for p, sp in zip(prompts, params):
            eng.add_request(p, sp)
        res = []
        while len(res) < len(prompts):
            res += eng.step()
        outs[flag] = {o.request_id: o for o in res}
        if flag == "1":
            assert not eng._groups and not eng._slot_group and int(eng.grp_pages.sum()) == 0 and int(eng.seq_skip.sum()) == 0
    same = 0
    for rid, a in outs["1"].items():
        b = outs["0"][rid]
        assert len(a.token_ids) == len(b.token_ids)
        n = next((i for i, (x, y) in enumerate(zip(a.token_ids, b.token_ids)) if x != y), len(a.token_ids))
        same += n == len(a.token_ids)
        assert max(abs(x - y) for x, y in zip(a.log_probs[: max(n, 1)], b.log_probs[: max(n, 1)])) < 5e-2
    assert same >= len(prompts) - 2
    assert int(ops.gemm_status()) == 0


def test_nvfp4_fake_quant_matches_reference():
    """NVFP4 fake-quantisation kernel against the plain PyTorch formulation of the same op (fp32 math)."""
    from verl_b200.utils.qat import nvfp4_fake_quantize, nvfp4_global_scale

    torch.manual_seed(0)
    x = (torch.randn(300, 1024, device="cuda") * 0.05).bfloat16()
    x[5] *= 40                                   # a row with large magnitudes (block scales near the top of e4m3)
    x[7, :32] = 0                                # all-zero blocks
    gs = nvfp4_global_scale(x)
    y = nvfp4_fake_quantize(x, gs)
    ref = nvfp4_fake_quantize(x.cpu().float(), gs)
    bad = (y.float().cpu() - ref).abs() > 1e-2 * ref.abs().clamp(min=1e-3)   # bf16 rounding of the output only
    assert bad.float().mean() < 1e-3, bad.float().mean()
    z = x.clone()
    nvfp4_fake_quantize(z, gs, out=z)            # in place
    assert torch.equal(z, y)


def test_fp8_grouped_expert_gemm_and_moe_layer(ops):
    """Grouped block-scaled fp8 GEMM against the same op on the host (dequantised fp32 product per 128-row tile), and the
    mixture-of-experts layer with fp8 expert copies against its bf16 result."""
    from verl_b200.models import DecoderModel, FlatParams
    from verl_b200.models.config import ModelConfig
    from verl_b200.ops import functional as F

    torch.manual_seed(0)
    E, N, K = 6, 384, 256
    counts = [130, 0, 128, 5, 250, 77]
    segs = [(c + 127) // 128 * 128 for c in counts]
    cap = sum(segs) + 256                                   # two unused tiles at the end
    x = torch.zeros(cap, K, device=DEV, dtype=torch.bfloat16)
    tile_expert, row = [], 0
    for e, (c, s_) in enumerate(zip(counts, segs)):
        x[row : row + c] = torch.randn(c, K, device=DEV).bfloat16()
        tile_expert += [e] * (s_ // 128)
        row += s_
    n_tiles = len(tile_expert)
    tile_expert += [E - 1] * (cap // 128 - n_tiles)
    te = torch.tensor(tile_expert, dtype=torch.int32, device=DEV)
    nt = torch.tensor([n_tiles], dtype=torch.int32, device=DEV)
    w = (torch.randn(E, N, K, device=DEV) * 0.05).bfloat16()
    wq, ws = F.fp8_quantize_1x128(w.reshape(E * N, K))
    y = F.linear_fp8_grouped(x, wq, ws, N, te, nt)
    # reference from the SAME quantised operands (host and device quantisers differ on rounding ties)
    xq, xs = F.fp8_quantize_1x128(x)
    xd = F.fp8_dequantize_1x128(xq.cpu(), xs.cpu())
    wd = F.fp8_dequantize_1x128(wq.cpu(), ws.cpu()).view(E, N, K)
    ref = torch.zeros(cap, N)
    for t in range(n_tiles):
        ref[t * 128 : (t + 1) * 128] = xd[t * 128 : (t + 1) * 128] @ wd[tile_expert[t]].t()
    assert ops.gemm_status() == 0
    assert rel(y, ref) < 1e-2
    assert rel(y, F.linear_fp8_grouped(x.cpu(), wq.cpu(), ws.cpu(), N, te.cpu(), nt.cpu()).float()) < 0.04  # host formulation of the op
    assert float(y[row:].abs().max()) == 0.0               # tiles beyond num_mtiles are not computed
    # layer level
    cfg = ModelConfig(model_type="qwen3_moe", vocab_size=512, hidden_size=256, intermediate_size=512, num_hidden_layers=1,
                      num_attention_heads=4, num_key_value_heads=2, head_dim=64, num_experts=16, num_experts_per_tok=4,
                      moe_intermediate_size=128, eos_token_id=2, pad_token_id=0)
    P = FlatParams(cfg, dtype=torch.bfloat16, device=DEV)
    P.init_weights(seed=4, std=0.05)
    model = DecoderModel(cfg, P)
    h2 = torch.randn(300, 256, device=DEV).bfloat16()
    ref_out = model._moe_fwd(P.layer(0), h2, None)
    assert model.quantize_linear_weights_fp8() > 0
    q_out = model._moe_fwd(P.layer(0), h2, None)
    assert ops.gemm_status() == 0
    assert 0 < rel(q_out, ref_out.float()) < 0.08           # fp8 operands: close to, not identical with, the bf16 layer


def test_rollout_engine_moe_cuda_graph_and_fp8_experts(ops):
    """Mixture-of-experts decoding under the CUDA graph equals eager decoding; with fp8 weight copies (dense projections and
    experts) generation runs and the sampled-token log-probs stay close to the bf16 engine's."""
    from verl_b200.models import FlatParams, ModelConfig
    from verl_b200.workers.rollout.native.engine import RolloutEngine, SamplingParams

    cfg = ModelConfig(model_type="qwen3_moe", vocab_size=2048, hidden_size=512, intermediate_size=1024, num_hidden_layers=2,
                      num_attention_heads=4, num_key_value_heads=2, head_dim=128, num_experts=16, num_experts_per_tok=4,
                      moe_intermediate_size=256, qk_norm=True, eos_token_id=-1, pad_token_id=0)
    P = FlatParams(cfg, dtype=torch.bfloat16, device=DEV)
    P.init_weights(seed=0, std=0.05)
    prompts = [[5, 6, 7, 8, 9], [10, 11, 12], [20, 21, 22, 23, 24, 25, 26], [3, 4]]
    outs = {}
    for key, graph, quant in (("graph", True, None), ("eager", False, None), ("fp8", True, "fp8")):
        eng = RolloutEngine(cfg, P, max_num_seqs=4, max_model_len=64, block_size=16, num_blocks=32, sync_interval=3,
                            use_cuda_graph=graph, eos_token_id=-1, quantization=quant)
        outs[key] = eng.generate(prompts, SamplingParams(temperature=0.0, max_tokens=8, logprobs=True))
    assert [o.token_ids for o in outs["graph"]] == [o.token_ids for o in outs["eager"]]
    assert all(len(o.token_ids) == 8 for o in outs["fp8"]) and ops.gemm_status() == 0
    # first generated token comes from the prefill (bf16 in both engines): identical; later ones may differ under fp8
    assert [o.token_ids[0] for o in outs["fp8"]] == [o.token_ids[0] for o in outs["graph"]]


def test_fp8_weight_block_quantiser_128x128(ops):
    from verl_b200.ops import functional as F

    torch.manual_seed(0)
    w = (torch.randn(300, 520, device=DEV) * 0.05).bfloat16()      # ragged: 3 x 5 blocks with partial edges
    w[130:140, 200:210] *= 30
    q, sc = F.fp8_quantize_128x128(w)
    q_c, sc_c = F.fp8_quantize_128x128(w.cpu())
    assert q.shape == (300, 520) and sc.shape == (3, 5)
    # identical scales; codes equal up to rounding ties (reciprocal multiply on the device, division on the host), and a
    # differing code is off by one step only
    assert rel(sc, sc_c) < 1e-6 and (q.cpu() != q_c).float().mean() < 3e-2
    assert rel(F.fp8_dequantize_128x128(q.cpu(), sc.cpu()), F.fp8_dequantize_128x128(q_c, sc_c)) < 1e-2
    assert rel(F.fp8_dequantize_128x128(q.cpu(), sc.cpu()), w.float()) < 0.07


def test_training_step_is_bitwise_reproducible_on_gpu(ops):
    """Deterministic mode: the same step run twice from the same seed gives identical bits (fixed reduction orders, no
    atomics on the training path)."""
    from functools import partial

    from verl_b200.models import get_preset
    from verl_b200.ops import functional as F
    from verl_b200.workers.config import FSDPEngineConfig, OptimizerConfig
    from verl_b200.workers.engine.native.engine import NativeEngineWithLMHead
    from verl_b200.workers.engine.utils import enable_full_determinism
    from verl_b200.workers.utils.losses import sft_loss

    saved = dict(F._ATTN_IMPL)
    try:
        def run():
            enable_full_determinism(11)
            eng = NativeEngineWithLMHead(get_preset("tiny-llama"), FSDPEngineConfig(seed=3, micro_batch_size_per_gpu=2), OptimizerConfig(lr=1e-2))
            eng.initialize()
            g = torch.Generator().manual_seed(5)
            ids = torch.randint(3, 500, (4, 96), generator=g).to(DEV)
            am = torch.ones_like(ids)
            data = {"input_ids": ids, "attention_mask": am, "responses": ids[:, -40:], "response_mask": am[:, -40:]}
            norms = [eng.train_batch(dict(data), partial(sft_loss, None))["metrics"]["grad_norm"] for _ in range(2)]
            return norms, eng.params.flat.clone()

        n1, w1 = run()
        n2, w2 = run()
        assert n1 == n2 and torch.equal(w1, w2)
    finally:
        F._ATTN_IMPL.update(saved)
        F.DETERMINISTIC_ATTENTION = False
        torch.use_deterministic_algorithms(False)
