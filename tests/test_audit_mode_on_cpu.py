"""Audit mode: index tensors are checked before an operator runs; off by default and free when off."""
import pytest
import torch

from verl_b200.ops import audit
from verl_b200.ops import functional as F


def test_audit_is_off_by_default_and_scoped():
    assert not audit.enabled()
    audit.check_index("op", "ids", torch.tensor([99]), 10)          # no-op when off
    with audit.scope():
        assert audit.enabled()
        with pytest.raises(audit.AuditError, match=r"op: ids has 2 value\(s\) outside \[0, 10\); first at flat position 1: 12"):
            audit.check_index("op", "ids", torch.tensor([[3, 12], [-1, 4]]), 10)
        audit.check_index("op", "slots", torch.tensor([-1, 4]), 10, skip_negative=True)
        with pytest.raises(audit.AuditError, match="integer tensor"):
            audit.check_index("op", "ids", torch.tensor([1.0]), 10)
    assert not audit.enabled()


def test_operators_refuse_bad_indices_before_running():
    w = torch.randn(16, 8)
    cos, sin = F.rope_table(32, 8, 1e4, "cpu")[:2] if isinstance(F.rope_table(32, 8, 1e4, "cpu"), tuple) else (None, None)
    with audit.scope():
        assert F.embedding(torch.tensor([0, 15]), w).shape == (2, 8)
        with pytest.raises(audit.AuditError, match="embedding: ids"):
            F.embedding(torch.tensor([0, 16]), w)
        with pytest.raises(audit.AuditError, match="embedding_bwd_: ids"):
            F.embedding_bwd_(torch.tensor([-1]), torch.zeros(1, 8), torch.zeros(16, 8))
        with pytest.raises(audit.AuditError, match="lmhead_logprob_entropy: labels"):
            F.lmhead_logprob_entropy(torch.randn(2, 8), w, torch.tensor([3, 16]))
        if cos is not None:
            x = torch.randn(3, 2, 8)
            F.apply_rope_(x, torch.tensor([0, 5, 31]), cos, sin)
            with pytest.raises(audit.AuditError, match="apply_rope_: positions"):
                F.apply_rope_(x, torch.tensor([0, 5, 32]), cos, sin)
        # paged cache: 4 blocks of 2 tokens, 1 KV head of size 8
        kc, vc = torch.zeros(4, 2, 1, 8), torch.zeros(4, 2, 1, 8)
        k, v = torch.randn(2, 1, 8), torch.randn(2, 1, 8)
        F.kv_append_(k, v, torch.tensor([7, -1]), kc, vc)                    # negative slot: skip, allowed
        with pytest.raises(audit.AuditError, match="kv_append_: slots"):
            F.kv_append_(k, v, torch.tensor([8, 0]), kc, vc)
        q = torch.randn(2, 2, 8)
        table = torch.tensor([[0, 1, 99], [2, 3, 0]])                         # 99 lies beyond the first sequence's context: unused
        assert F.paged_decode_attention(q, kc, vc, table, torch.tensor([4, 5])).shape == (2, 2, 8)
        with pytest.raises(audit.AuditError, match="block_table"):
            F.paged_decode_attention(q, kc, vc, table, torch.tensor([5, 5]))   # now the context reaches entry 99
        with pytest.raises(audit.AuditError, match="ctx_len"):
            F.paged_decode_attention(q, kc, vc, table, torch.tensor([4, 7]))   # longer than three blocks hold
    # off: the same bad call is not checked here (the CPU reference then fails in its own way or not at all)
    assert F.embedding(torch.tensor([0, 15]), w).shape == (2, 8)


def test_alignment_check():
    base = torch.zeros(64, dtype=torch.bfloat16)
    with audit.scope():
        audit.check_aligned("op", "x", base[:32].view(2, 16))
        with pytest.raises(audit.AuditError, match="not a multiple of 16 bytes"):
            audit.check_aligned("op", "x", base[1:33])
        with pytest.raises(audit.AuditError, match="rows of x are 6 bytes apart"):
            audit.check_aligned("op", "x", base[:6].view(2, 3))
