"""AdamW with block-quantised moments: ``adamw8bit``, ``adamw4bit``, ``adamwfp8``.

The reference registers these three names from an optional third-party package
(src/kohakuwullm/training/optim/torchao_optim.py:12-31: "quantizes the Adam moments only"). Here they are one
optimizer of this framework's own. Parameters and the update arithmetic stay in fp32 (or the parameter's
dtype with fp32 arithmetic); only ``exp_avg`` and ``exp_avg_sq`` are held quantised between steps, in blocks
of ``block`` elements with one fp32 scale per block:

* ``int8``  -- 8-bit codes of a square-root companded value (``sign(x) sqrt(|x| / absmax)``), which spends the
  codes on the small magnitudes where most of a moment's mass sits; 1 byte + 4/block bytes per element.
* ``int4``  -- the same on 4-bit codes, two per byte, block 128; the second moment uses a fourth-root companding
  there and never rounds a non-zero value to zero (a zero second moment would turn its element's update into
  ``m / eps``).
* ``fp8``   -- ``float8_e4m3fn`` values scaled so that the block's absmax maps to 448.

Per element the state costs 2.03 bytes (8-bit, fp8) or 1.06 bytes (4-bit) instead of 8. Every step dequantises
a parameter's moments, does the AdamW update in fp32 and quantises them again; tensors smaller than
``min_quantized_size`` keep fp32 moments (norm gains and biases are tiny and sensitive).
"""

from __future__ import annotations

import torch

FORMATS = ("int8", "int4", "fp8")


def _blocks(x: torch.Tensor, block: int) -> torch.Tensor:
    flat = x.reshape(-1)
    pad = (-flat.numel()) % block
    if pad:
        flat = torch.cat([flat, flat.new_zeros(pad)])
    return flat.view(-1, block)


def _power(fmt: str, signed: bool) -> float:
    return 0.25 if (fmt == "int4" and not signed) else 0.5


def quantize_blocks(x: torch.Tensor, fmt: str, block: int, signed: bool) -> dict:
    """fp32 tensor -> {"codes", "scale"}. ``signed`` False: the values are non-negative (second moment)."""
    b = _blocks(x.float(), block)
    scale = b.abs().amax(dim=1, keepdim=True).clamp(min=1e-30)
    if fmt == "fp8":
        codes = (b * (448.0 / scale)).to(torch.float8_e4m3fn)
        return {"codes": codes, "scale": scale.squeeze(1)}
    levels = {"int8": (127 if signed else 255), "int4": (7 if signed else 15)}[fmt]
    y = (b.abs() / scale) ** _power(fmt, signed)      # companded magnitude in [0, 1]
    q = torch.round(y * levels)
    if signed:
        q = q * torch.sign(b) + levels                # 0 .. 2 * levels
    else:
        q = torch.where((b > 0) & (q < 1), torch.ones_like(q), q)
    q = q.to(torch.uint8)
    if fmt == "int4":
        q = q[:, 0::2] | (q[:, 1::2] << 4)
    return {"codes": q, "scale": scale.squeeze(1)}


def dequantize_blocks(packed: dict, fmt: str, block: int, signed: bool, shape: torch.Size) -> torch.Tensor:
    codes, scale = packed["codes"], packed["scale"].unsqueeze(1)
    if fmt == "fp8":
        out = codes.float() * (scale / 448.0)
    else:
        levels = {"int8": (127 if signed else 255), "int4": (7 if signed else 15)}[fmt]
        if fmt == "int4":
            q = torch.stack([codes & 0xF, codes >> 4], dim=2).reshape(codes.shape[0], -1)
        else:
            q = codes
        q = q.float()
        inv = 1.0 / _power(fmt, signed)
        if signed:
            q = q - levels
            out = torch.sign(q) * (q.abs() / levels) ** inv * scale
        else:
            out = (q / levels) ** inv * scale
    n = 1
    for d in shape:
        n *= d
    return out.reshape(-1)[:n].view(shape)


class QuantizedStateAdamW(torch.optim.Optimizer):
    def __init__(self, params, lr=3e-4, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1, state_format: str = "int8",
                 block: int | None = None, min_quantized_size: int = 4096):
        if state_format not in FORMATS:
            raise ValueError(f"state_format must be one of {FORMATS}, not {state_format!r}")
        super().__init__(params, dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay))
        self.fmt = state_format
        self.block = block or (128 if state_format == "int4" else 256)
        if self.block % 2:
            raise ValueError("block must be even")
        self.min_quantized_size = min_quantized_size

    def _load(self, st: dict, key: str, signed: bool, shape) -> torch.Tensor:
        v = st[key]
        return dequantize_blocks(v, self.fmt, self.block, signed, shape) if isinstance(v, dict) else v

    def _store(self, st: dict, key: str, value: torch.Tensor, signed: bool, quantised: bool) -> None:
        st[key] = quantize_blocks(value, self.fmt, self.block, signed) if quantised else value

    @torch.no_grad()
    def step(self, closure=None):
        loss = closure() if closure is not None else None
        for group in self.param_groups:
            b1, b2 = group["betas"]
            for p in group["params"]:
                if p.grad is None:
                    continue
                st = self.state[p]
                quantised = p.numel() >= self.min_quantized_size
                if not st:
                    st["step"] = 0
                    zeros = torch.zeros(p.shape, dtype=torch.float32, device=p.device)
                    self._store(st, "exp_avg", zeros, True, quantised)
                    self._store(st, "exp_avg_sq", zeros.clone(), False, quantised)
                st["step"] += 1
                g = p.grad.float()
                m = self._load(st, "exp_avg", True, p.shape).mul_(b1).add_(g, alpha=1 - b1)
                v = self._load(st, "exp_avg_sq", False, p.shape).mul_(b2).addcmul_(g, g, value=1 - b2)
                bc1, bc2 = 1 - b1 ** st["step"], 1 - b2 ** st["step"]
                update = (m / bc1) / ((v / bc2).sqrt() + group["eps"])
                new = p.float() * (1 - group["lr"] * group["weight_decay"]) - group["lr"] * update
                p.copy_(new.to(p.dtype))
                self._store(st, "exp_avg", m, True, quantised)
                self._store(st, "exp_avg_sq", v, False, quantised)
        return loss

    def state_bytes(self) -> int:
        """Bytes held by the moments (codes + scales), for memory accounting."""
        total = 0
        for st in self.state.values():
            for key in ("exp_avg", "exp_avg_sq"):
                v = st.get(key)
                if isinstance(v, dict):
                    total += v["codes"].numel() * v["codes"].element_size() + v["scale"].numel() * 4
                elif v is not None:
                    total += v.numel() * v.element_size()
        return total
