"""Tutorial 04 - expert-parallel all-to-all for MoE inference (DeepSeek-style dispatch / combine).

    torchrun --nproc-per-node 4 tutorials/04-deepseek-infer-all2all.py

Each rank holds 128 tokens with top-8 routing over 64 experts, experts sharded over the ranks.  ``ep_dispatch`` sends
every (token, slot) to the owner of its expert in one kernel: rows are quantised to fp8 (e4m3, one scale per 128
values) on the way out, written straight into the receiver's buffer over NVLink, and arrive sorted by local expert and
padded to 128-row tiles for the grouped GEMM.  ``ep_combine`` returns the expert outputs and applies the routing
weights while it sums the k slots.  Reference: tutorials/04-deepseek-infer-all2all.py and
kernels/nvidia/low_latency_all_to_all.py (137 us for this shape on 32 H800, README.md:94).
"""
import torch
from _common import done, say, start

from triton_distributed_b200 import ops

rt = start()
W = rt.world_size
T, H, E, K = 128, 1024, 16 * W, 8
x = torch.randn(T, H, device=rt.device).to(torch.bfloat16)
logits = torch.randn(T, E, device=rt.device)
topk_w, topk_ids = torch.softmax(logits, -1).topk(K, dim=-1)
topk_w = (topk_w / topk_w.sum(-1, keepdim=True)).float()

ctx = ops.create_all_to_all_context(max_m=T, hidden=H, num_tot_experts=E, topk=K, quant=True, layout="ll")
recv = ops.ep_dispatch(ctx, x, topk_ids)
# an "expert" that just scales by (local expert id + 1) keeps the check simple: the grouped GEMM goes here
y = recv.x_sorted.clone()
out = ops.ep_combine(ctx, y, recv, topk_w)

# identity experts: the weighted sum of k copies of a token is the token itself (up to the fp8 round trip)
err = (out.float() - x.float()).abs().max().item() / x.float().abs().max().item()
assert err < 0.08, err
say(rt, f"dispatch -> identity experts -> combine returns the tokens (fp8 round trip, rel err {err:.3f})")
ctx.finalize()
done(rt, "04-ep-all2all")
