"""Ulysses and ring attention over host-engine communicators (ranks as threads, CPU tensors) against plain attention
over the whole sequence."""
import math

import pytest
import torch
import torch.nn.functional as F

import hccl_b200 as hb
from hccl_b200 import Communicator
from hccl_b200.parallel import ring_attention, ulysses_attention

from test_host_engine import run_ranks


def reference(q, k, v, causal):
    o = F.scaled_dot_product_attention(q.transpose(0, 1).double(), k.transpose(0, 1).double(), v.transpose(0, 1).double(), is_causal=causal,
                                       scale=1.0 / math.sqrt(q.shape[-1]))
    return o.transpose(0, 1)


@pytest.mark.parametrize("fn", [ulysses_attention, ring_attention], ids=["ulysses", "ring"])
@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("P", [1, 2, 4])
def test_sequence_sharded_attention_matches_full_attention(fn, causal, P):
    torch.manual_seed(3)
    S, H, D = 32 * P, 8, 16
    q, k, v = (torch.randn(S, H, D) for _ in range(3))
    want = reference(q, k, v, causal)
    comms = Communicator.host_sim(P, None, hb.make_config(buffer_mib=8, exec_timeout_ms=20000))
    outs = [None] * P
    s = S // P

    def body(r, c):
        sl = slice(r * s, (r + 1) * s)
        outs[r] = fn(q[sl].contiguous(), k[sl].contiguous(), v[sl].contiguous(), c, causal=causal)

    run_ranks(comms, body)
    got = torch.cat(outs)
    torch.testing.assert_close(got.double(), want, rtol=1e-4, atol=1e-5)
    for c in comms:
        c.destroy()


def test_ulysses_rejects_heads_that_do_not_divide():
    comms = Communicator.host_sim(3)
    x = torch.randn(4, 8, 16)
    with pytest.raises(ValueError):
        ulysses_attention(x, x, x, comms[0])
    for c in comms:
        c.destroy()
