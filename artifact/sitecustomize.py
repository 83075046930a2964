"""Start-up hook for the TorchTitan baseline of the evaluation (picked up when ``artifact/`` is on PYTHONPATH).

With ``TORCHTITAN_USE_BMM_EXPERTS=1`` TorchTitan's grouped-expert forward is replaced by the padded
batched-matmul formulation the reference's own expert op uses (every expert padded to the largest token count,
three ``bmm`` calls), so that the baseline and the reference run the same expert arithmetic.  This framework
itself never uses that formulation: its experts are ragged grouped tcgen05 GEMMs.  Counterpart of the
reference's ``artifact/sitecustomize.py:1-64``.
"""
import os


def _padded_bmm_experts(w1, w2, w3, x, counts):
    import torch
    import torch.nn.functional as F

    counts = counts.to(device=x.device, dtype=torch.long)
    experts, dim = w1.shape[0], x.shape[-1]
    cap = int(counts.max()) if counts.numel() else 0
    first = torch.cumsum(counts, 0) - counts
    slot = torch.arange(cap, device=x.device)
    valid = slot[None, :] < counts[:, None]                      # [E, cap]
    src = (first[:, None] + slot[None, :]).clamp_(max=max(x.shape[0] - 1, 0))
    packed = torch.where(valid[..., None], x[src], x.new_zeros(()))   # [E, cap, dim]
    h = F.silu(torch.bmm(packed, w1.transpose(1, 2))) * torch.bmm(packed, w3.transpose(1, 2))
    y = torch.bmm(h, w2.transpose(1, 2))
    out = x.new_zeros(x.shape)
    out.index_add_(0, src[valid], y[valid])
    assert out.shape[-1] == dim and w1.shape[0] == experts
    return out


if os.environ.get("TORCHTITAN_USE_BMM_EXPERTS") == "1":
    try:
        from torch.distributed.tensor import DTensor
        from torchtitan.models.common.moe import moe as _moe

        def _forward(self, x, num_tokens_per_expert):
            ws = [w.to_local() if isinstance(w, DTensor) else w for w in (self.w1, self.w2, self.w3)]
            return _padded_bmm_experts(*ws, x, num_tokens_per_expert)

        _moe.GroupedExperts.forward = _forward
        print("[artifact] TorchTitan GroupedExperts.forward -> padded bmm experts", flush=True)
    except Exception as exc:  # pragma: no cover - depends on an optional package
        raise RuntimeError("could not install the TorchTitan bmm-experts hook") from exc
