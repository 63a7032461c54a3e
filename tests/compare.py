"""How the engine's logits are compared with the plain implementation's: the largest difference of a position
against that row's largest |logit|, top-1 agreement outside near-ties, and the mean KL divergence -- the figures
the reference's trace comparison reports (scripts/compare-traces.ts:59-80)."""
from typing import Dict

import torch

# float32: both sides compute in float with different summation orders.
# bfloat16: the plain side rounds where the engine stores; what is left is the order of summation and where a
# fused kernel rounds. Observed on a B200: float32 up to 1.5e-6 of a row's largest |logit| (3.1e-6 at the 0.5B layer
# sizes), mean KL below 1e-12; bfloat16 up to 0.75 % at the tiny sizes and 0.94 % at the 0.5B layer sizes, where the
# maximum is taken over 151,936 logits a row (hence REL_WIDE there), mean KL up to 2e-6 (1e-5 at the 0.5B sizes).
REL = {"float32": 5e-6, "bfloat16": 1e-2}
REL_WIDE = {"float32": 5e-6, "bfloat16": 1.5e-2}
MEAN_KL = {"float32": 1e-9, "bfloat16": 3e-5}


def figures(got: torch.Tensor, want: torch.Tensor):
    """(worst |difference| / row's largest |logit|, its position, top-1 agreement outside near-ties, mean KL)."""
    got, want = got.double(), want.double()
    scale = want.abs().max(dim=1).values.clamp_min(1e-6)
    rel = (got - want).abs().max(dim=1).values / scale
    top2 = want.topk(2, dim=1).values
    clear = (top2[:, 0] - top2[:, 1]) > 2 * (got - want).abs().max(dim=1).values     # rounding cannot swap these
    same = got.argmax(dim=1) == want.argmax(dim=1)
    agree = float(same[clear].double().mean()) if bool(clear.any()) else 1.0
    lw, lg = torch.log_softmax(want, dim=1), torch.log_softmax(got, dim=1)
    kl = float((lw.exp() * (lw - lg)).sum(dim=1).mean())
    return float(rel.max()), int(rel.argmax()), agree, kl


def check_logits(got: Dict[str, torch.Tensor], want: Dict[str, torch.Tensor], dtype: str, what: str, bound=None) -> None:
    bound = (bound or REL)[dtype]
    for rid in want:
        assert got[rid].shape == want[rid].shape, f"{what} {rid}: shape {tuple(got[rid].shape)} vs {tuple(want[rid].shape)}"
        worst, at, agree, kl = figures(got[rid], want[rid])
        rel = (got[rid] - want[rid]).abs().max(dim=1).values / want[rid].abs().max(dim=1).values.clamp_min(1e-6)
        assert worst <= bound, f"{what} {rid}: first position over the bound {int((rel > bound).nonzero()[0])}, " \
            f"worst {worst:.3g} of the row's largest logit at position {at} of {len(rel)}"
        assert agree == 1.0, f"{what} {rid}: top-1 agreement {agree:.4f} outside near-ties"
        assert kl <= MEAN_KL[dtype], f"{what} {rid}: mean KL {kl:.3g}"
