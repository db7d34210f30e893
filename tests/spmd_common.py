"""Builders shared by the SPMD-program tests (CPU and GPU)."""
import copy
from types import SimpleNamespace

import torch
import torch.nn.functional as F

from hap_b200 import plan as P

RATIOS = [0.6, 0.4]
BATCH, IN, HID, OUT = 64, 1024, 4096, 1024


def reference_model(dtype=torch.float32, small=False):
    torch.manual_seed(39)                       # the reference's model seed (worker.py:20)
    dims = (64, 136, 72) if small else (IN, HID, OUT)
    return P.MLP(*dims).to(dtype), dims


def batch(dims, dtype=torch.float32, n=BATCH):
    g = torch.Generator().manual_seed(2024)
    return torch.randn(n, dims[0], generator=g).to(dtype), torch.randn(n, dims[2], generator=g).to(dtype)


def rank_modules(model, plan, ns, world=2, device="cpu"):
    mods = []
    for r in range(world):
        m = copy.deepcopy(model)
        graph = P.emit_mlp(m, plan, RATIOS, r, BATCH, ns)
        mods.append(torch.fx.GraphModule(m, graph).to(device))
    return mods


def cpu_namespace():
    from oracle import gloo_port
    return SimpleNamespace(collectives=gloo_port, linear=F.linear)


def full_gradients(model, x, y):
    m = copy.deepcopy(model).double()
    loss = m(x.double(), y.double())
    loss.backward()
    return float(loss), {n: p.grad.clone() for n, p in m.named_parameters()}


def expected_shard(full, name, plan, rank, dims):
    """What rank `rank` must hold for the full-model gradient `full` of parameter `name`."""
    if plan == "dp":
        return full
    from hap_b200 import sharding_round
    extent = dims[1] if name.startswith("fc1") else dims[2]
    return torch.split(full, sharding_round(extent, RATIOS), dim=0)[rank]


# ---- Transformer language model ------------------------------------------------------------------
LM_SMALL = dict(vocab=64, d_model=64, nheads=2, d_ffn=128, nlayers=2, seqlen=16)
LM_BATCH = 8


def lm_model(dtype=torch.float32):
    torch.manual_seed(39)
    return P.TransformerLM(**LM_SMALL).to(dtype)


def lm_batch():
    g = torch.Generator().manual_seed(2024)
    return (torch.randint(0, LM_SMALL["vocab"], (LM_BATCH, LM_SMALL["seqlen"]), generator=g),
            torch.randint(0, LM_SMALL["vocab"], (LM_BATCH, LM_SMALL["seqlen"]), generator=g))


def lm_rank_modules(model, plan, ns, world=2, device="cpu"):
    mods = []
    for r in range(world):
        m = copy.deepcopy(model).to(device)
        graph = P.emit_lm(m, plan, RATIOS, r, LM_BATCH, ns)
        mods.append(torch.fx.GraphModule(m, graph))
    return mods


def lm_cpu_namespace():
    from oracle import gloo_port
    return SimpleNamespace(collectives=gloo_port, linear=F.linear, mha=F.multi_head_attention_forward)


# ---- Vision Transformer ------------------------------------------------------------------------------
VIT_SMALL = dict(image=16, patch=4, channels=3, d_model=64, nheads=2, d_ffn=128, nlayers=2, nclasses=10)


def vit_model(dtype=torch.float32):
    torch.manual_seed(39)
    return P.ViT(**VIT_SMALL).to(dtype)


def vit_batch(dtype=torch.float32):
    g = torch.Generator().manual_seed(2024)
    return (torch.randn(LM_BATCH, VIT_SMALL["channels"], VIT_SMALL["image"], VIT_SMALL["image"], generator=g).to(dtype),
            torch.randint(0, VIT_SMALL["nclasses"], (LM_BATCH,), generator=g))


def vit_rank_modules(model, plan, ns, world=2, device="cpu", ratios=None):
    mods = []
    for r in range(world):
        m = copy.deepcopy(model).to(device)
        mods.append(torch.fx.GraphModule(m, P.emit_vit(m, plan, ratios or RATIOS, r, LM_BATCH, ns)))
    return mods


# ---- MoE Transformer ---------------------------------------------------------------------------------
MOE_SMALL = dict(vocab=64, d_model=64, nheads=2, d_ffn=128, nlayers=2, seqlen=16, n_expert=4, capacity=8)


def moe_model(dtype=torch.float32):
    torch.manual_seed(39)
    return P.MoETransformerLM(**MOE_SMALL).to(dtype)


def moe_rank_modules(model, ns, world=2, device="cpu", ratios=None):
    mods = []
    for r in range(world):
        m = copy.deepcopy(model).to(device)
        mods.append(torch.fx.GraphModule(m, P.emit_moe(m, ratios or RATIOS, r, LM_BATCH, ns)))
    return mods


def moe_cpu_namespace():
    from oracle import gloo_port
    return SimpleNamespace(collectives=gloo_port, linear=F.linear, mha=F.multi_head_attention_forward, einsum=torch.einsum)
