"""AdamW with 8-bit optimizer state for the parameters Muon does not take (scalars, norms, embeddings, the output layer),
or for every parameter (``--optimizer adam8bit``).

State per 256-element block, with ``am_m = max |m|`` and ``am_v = max sqrt(v)`` in fp32: ``m8 = round(127 sign(m)
sqrt(|m| / am_m))`` (int8) and ``v8 = round(255 sqrt(sqrt(v) / am_v))`` (uint8) - square-root companded codes, so the small
entries of a block keep relative precision; 2 bytes per parameter instead of 8.  The reference selects this optimizer for the non-matrix
parameters of its Muon lanes (``muon_scalar_optimizer = "adam8bit"``, cppmega/recipes/run_profiles.py:181) and takes the
implementation from Megatron's emerging-optimizers fork; this file is the definition (PyTorch) and the front door of the
kernel in ``ops/csrc/qmuon.cu``.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import Optional

import torch

QBLOCK = 256


@dataclass
class Adam8bitState:
    m8: torch.Tensor          # int8 [n]
    v8: torch.Tensor          # uint8 [n]
    am_m: torch.Tensor        # fp32 [ceil(n / 256)]
    am_v: torch.Tensor        # fp32 [ceil(n / 256)]

    @classmethod
    def zeros(cls, n: int, device) -> "Adam8bitState":
        nb = (n + QBLOCK - 1) // QBLOCK
        return cls(torch.zeros(n, dtype=torch.int8, device=device), torch.zeros(n, dtype=torch.uint8, device=device),
                   torch.zeros(nb, dtype=torch.float32, device=device), torch.zeros(nb, dtype=torch.float32, device=device))

    def moments(self):
        """Dequantised (m, v) as fp32."""
        n = self.m8.numel()
        sm = (self.am_m / (127.0 * 127.0)).repeat_interleave(QBLOCK)[:n]
        sv = (self.am_v / (255.0 * 255.0)).repeat_interleave(QBLOCK)[:n]
        qm, qv = self.m8.float(), self.v8.float()
        r = qv * qv * sv
        return qm * qm.abs() * sm, r * r

    def nbytes(self) -> int:
        return 2 * self.m8.numel() + 8 * self.am_m.numel()


def adam8bit_reference(master, st: Adam8bitState, g, out, wd_mask, clip, lr, b1, b2, eps, wd, bc1, bc2,
                       active: Optional[torch.Tensor] = None) -> None:
    """Definition the kernel is tested against (same arithmetic, fp32)."""
    n = master.numel()
    nb = (n + QBLOCK - 1) // QBLOCK
    m_old, v_old = st.moments()
    gf = g.float() * clip
    on = torch.ones(n, dtype=torch.bool, device=master.device) if active is None else active.bool()
    m = torch.where(on, b1 * m_old + (1.0 - b1) * gf, m_old)
    v = torch.where(on, b2 * v_old + (1.0 - b2) * gf * gf, v_old)
    upd = (m / bc1) / ((v / bc2).sqrt() + eps) + wd * master * wd_mask.to(master.dtype)
    master.copy_(torch.where(on, master - lr * upd, master))
    out.copy_(torch.where(on, master.to(out.dtype), out))
    pad = nb * QBLOCK - n
    mp = torch.nn.functional.pad(m, (0, pad)).view(nb, QBLOCK)
    rp = torch.nn.functional.pad(v.sqrt(), (0, pad)).view(nb, QBLOCK)
    am_m, am_v = mp.abs().amax(-1), rp.amax(-1)
    im = torch.where(am_m > 0, 1.0 / am_m, torch.zeros_like(am_m)).unsqueeze(-1)
    ir = torch.where(am_v > 0, 1.0 / am_v, torch.zeros_like(am_v)).unsqueeze(-1)
    qa = torch.floor(127.0 * (mp.abs() * im).sqrt() + 0.5).clamp(max=127)
    st.m8.copy_((torch.sign(mp) * qa).to(torch.int8).view(-1)[:n])
    st.v8.copy_(torch.floor(255.0 * (rp * ir).sqrt() + 0.5).clamp(0, 255).to(torch.uint8).view(-1)[:n])
    st.am_m.copy_(am_m)
    st.am_v.copy_(am_v)


def adam8bit_update(master, st: Adam8bitState, g, out, wd_mask, clip, lr, b1, b2, eps, wd, bc1, bc2,
                    active: Optional[torch.Tensor] = None, gate: Optional[torch.Tensor] = None) -> None:
    """One step on a flat fp32 master shard; writes the low-precision copy into ``out``.  ``active`` (bool / uint8 per
    element): elements with 0 are left alone.  ``gate`` (CUDA): device word, non-zero skips the whole update."""
    gk = {torch.float32: 0, torch.bfloat16: 1}.get(g.dtype)
    ok = {torch.float32: 0, torch.bfloat16: 1}.get(out.dtype)
    if master.is_cuda and gk is not None and ok is not None:
        from ..ops import cuda as cu
        from ..ops import functional as F_
        L = cu.lib()
        if not getattr(L, "_a8_declared", False):
            vp, i32, i64, f32 = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float
            L.cm_adam8bit.argtypes = [vp] * 10 + [i64] + [f32] * 7 + [i32, i32, vp, vp]
            L.cm_adam8bit.restype = i32
            L._a8_declared = True
        clip_t = (clip if torch.is_tensor(clip) else torch.tensor(float(clip), device=master.device)).reshape(1).float()
        act = None if active is None else active.to(torch.uint8).contiguous()
        rc = L.cm_adam8bit(master.data_ptr(), st.m8.data_ptr(), st.v8.data_ptr(), st.am_m.data_ptr(), st.am_v.data_ptr(),
                           g.data_ptr(), out.data_ptr(), wd_mask.data_ptr(), None if act is None else act.data_ptr(),
                           clip_t.data_ptr(), master.numel(), float(lr), float(b1), float(b2), float(eps), float(wd),
                           float(bc1), float(bc2), gk, ok, None if gate is None else gate.data_ptr(), cu.stream_ptr())
        if rc:
            raise RuntimeError(f"cm_adam8bit failed ({rc})")
        F_.count_launch("adam8bit")
        return
    adam8bit_reference(master, st, g, out, wd_mask, clip, lr, b1, b2, eps, wd, bc1, bc2, active)
