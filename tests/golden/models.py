"""Small torch models shared by the fixture generator and the tests."""

import torch
from torch import nn


class TinyGatedLM(nn.Module):
    """Embedding -> 2 x (residual Linear, gated MLP with up * act(gate) -> down) -> head: the layer kinds and
    the Linear -> multiply -> Linear pattern of a Llama decoder at toy size."""

    def __init__(self, vocab=64, hidden=32, inter=64, layers=2, seed=0):
        super().__init__()
        g = torch.Generator().manual_seed(seed)
        self.embed = nn.Embedding(vocab, hidden)
        self.blocks = nn.ModuleList()
        for _ in range(layers):
            blk = nn.ModuleDict({"q": nn.Linear(hidden, hidden, bias=False), "gate": nn.Linear(hidden, inter, bias=False),
                                 "up": nn.Linear(hidden, inter, bias=False), "down": nn.Linear(inter, hidden, bias=False)})
            self.blocks.append(blk)
        self.head = nn.Linear(hidden, vocab, bias=False)
        with torch.no_grad():
            for p in self.parameters():
                p.copy_(torch.randn(p.shape, generator=g) * 0.1)
            # a few outlier channels so that AWQ has something to do
            self.embed.weight[:, :2] *= 8.0

    def forward(self, ids):
        x = self.embed(ids)
        for blk in self.blocks:
            h = x + blk["q"](x)
            x = h + blk["down"](torch.nn.functional.silu(blk["gate"](h)) * blk["up"](h))
        return self.head(x)


class StackedLinear(nn.Module):
    """n stacked Linear(width -> width, bias=False) layers with N(0, 0.02^2) weights from seed 0: with 8 layers
    of width 4096 in fp32 this is the CPU-runnable benchmark configuration of the compression path."""

    def __init__(self, n_layers: int = 8, width: int = 4096, seed: int = 0):
        super().__init__()
        self.width = width
        self.layers = nn.ModuleList(nn.Linear(width, width, bias=False) for _ in range(n_layers))
        g = torch.Generator().manual_seed(seed)
        with torch.no_grad():
            for lin in self.layers:
                lin.weight.copy_(torch.randn(lin.weight.shape, generator=g) * 0.02)

    def forward(self, x):
        for lin in self.layers:
            x = lin(x)
        return x

    def example_input(self):
        return torch.randn(1, self.width, generator=torch.Generator().manual_seed(1))


def calibration_ids(n=6, seq=16, vocab=64, seed=1):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, vocab, (1, seq), generator=g) for _ in range(n)]


API_CASES = [
    # name, kwargs (mode etc.), uses dataset
    ("int8_asym_default", dict(mode="int8_asym"), False),
    ("int8_sym", dict(mode="int8_sym"), False),
    ("int4_sym_g16", dict(mode="int4_sym", group_size=16), False),
    ("int4_asym_g16_all", dict(mode="int4_asym", group_size=16, all_layers=True), False),
    ("int4_sym_g16_ratio", dict(mode="int4_sym", group_size=16, ratio=0.6), False),
    ("int4_asym_g16_ratio_maxvar", dict(mode="int4_asym", group_size=16, ratio=0.6,
                                        sensitivity_metric="max_activation_variance"), True),
    ("int4_sym_g16_ratio_hessian", dict(mode="int4_sym", group_size=16, ratio=0.5,
                                        sensitivity_metric="hessian_input_activation"), True),
    ("int4_sym_g16_ratio_meanvar", dict(mode="int4_sym", group_size=16, ratio=0.7,
                                        sensitivity_metric="mean_activation_variance"), True),
    ("int4_asym_g16_ratio_meanmag", dict(mode="int4_asym", group_size=16, ratio=0.4,
                                         sensitivity_metric="mean_activation_magnitude"), True),
    ("int4_asym_g16_se", dict(mode="int4_asym", group_size=16, scale_estimation=True), True),
    ("int4_sym_g16_awq", dict(mode="int4_sym", group_size=16, awq=True), True),
    ("int4_asym_g16_awq_se", dict(mode="int4_asym", group_size=16, awq=True, scale_estimation=True), True),
]


# model-level GPTQ fixture: a toy decoder wide enough that every Hessian has more tokens than channels
LAYERWISE = dict(model=dict(vocab=64, hidden=128, inter=256, layers=2, seed=3), group_size=32, block=128, damp=0.1,
                 modes=("int4_sym", "int4_asym"), n=8, seq=64)


def layerwise_ids():
    return calibration_ids(n=LAYERWISE["n"], seq=LAYERWISE["seq"], vocab=LAYERWISE["model"]["vocab"], seed=7)
