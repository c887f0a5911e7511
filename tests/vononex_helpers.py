"""Shared by the Vononex tests: small configurations that differ from one another in every size and constant
(head counts, shared key/value heads, key and value sizes that differ, partly rotated heads, layers without a
feed-forward, widths the tensor-core kernels refuse), model folders with seeded random weights, trace builders
and the comparison with the plain implementation (tests/plain/vononex_plain.py)."""
from __future__ import annotations

import copy
import os
import tempfile

import torch

from plain import vononex_plain as VP


def parallel(left, right, left_scale, right_scale, ff):
    return {"type": "parallel", "mixer": {"left": left, "right": right, "left_scale": left_scale,
                                          "right_scale": right_scale},
            "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def mingru(width, ff):
    return {"type": "mingru", "mixer": {"width": width}, "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def left(heads, kv, dim, vdim, scale, rot_dims, base):
    return {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale, "rot": {"dims": rot_dims, "base": base}}


def right(heads, dim, vdim, decay, rot_dims, base):
    return {"heads": heads, "dim": dim, "vdim": vdim, "decay": decay, "rot": {"dims": rot_dims, "base": base}}


# Odd sizes everywhere: a recurrent first layer without feed-forward, 6 heads on 2 key/value heads with keys of 24
# and values of 40, rotations over a part of the head, a retention whose key size is no multiple of four and whose
# values are narrower than a block of the scan, an inner width that the tensor-core product refuses.
CONFIG_P = {"architecture": "Vononex", "vocab": 211, "width": 72, "postln_alpha": 1.7, "norm": {"eps": 1e-4},
            "init_std": 0.25, "layers": [
                mingru(40, None),
                parallel(left(6, 2, 24, 40, 0.3, 16, 500.0), right(3, 20, 24, [0.9, 0.97, 0.995], 12, 10000.0), 0.7, 1.3, 88),
                parallel(left(2, 1, 64, 32, 0.125, 64, 10000.0), right(2, 18, 10, [0.5, 0.9999], 6, 77.0), 1.1, 0.4, 50),
                mingru(33, 64)]}
# Sizes the tensor-core kernels take: head sizes 128 and 64 (and 32 beside 96, stored as 96), several key/value
# heads, retention with 128 rows a column.
CONFIG_Q = {"architecture": "Vononex", "vocab": 1003, "width": 320, "postln_alpha": 3.0, "norm": {"eps": 1e-6},
            "init_std": 0.12, "layers": [
                parallel(left(4, 2, 128, 128, 0.09, 128, 20000.0), right(2, 128, 64, [0.96875, 0.999], 64, 5e5), 1.3, 0.7, 384),
                mingru(448, 192),
                parallel(left(4, 4, 64, 64, 0.125, 32, 1e5), right(4, 32, 32, [0.9, 0.99, 0.995, 0.9995], 32, 3e4), 0.8, 1.0, None),
                parallel(left(3, 1, 32, 96, 0.2, 32, 3e4), right(1, 256, 16, [0.98], 256, 7e3), 1.0, 1.5, 128)]}
# A width and a vocabulary that are no multiples of 8 (the 16-bit engine falls back to the CUDA-core product and to
# scalar loads everywhere), as many key/value heads as heads, head sizes of 20, a feed-forward narrower than the model.
CONFIG_R = {"architecture": "Vononex", "vocab": 333, "width": 100, "postln_alpha": 0.8, "norm": {"eps": 1e-5},
            "init_std": 0.2, "layers": [
                parallel(left(5, 5, 20, 20, 0.22, 20, 2000.0), right(5, 20, 20, [0.8, 0.9, 0.95, 0.99, 0.999], 20, 2000.0), 1.0, 1.0, 36),
                mingru(100, None),
                parallel(left(2, 1, 50, 30, 0.14, 10, 50.0), right(1, 100, 100, [0.97], 0, 1.0), 0.5, 2.0, 70)]}
CONFIGS = {"P": CONFIG_P, "Q": CONFIG_Q, "R": CONFIG_R}

# float32: both sides differ by the order of additions only; every row is held to this.
# bfloat16: activations are rounded to 8 bits of mantissa between kernels, and these small random models pass
# that noise on unevenly (measured: 10^4 times the float32 error row by row, median 1.4-2.3e-2, a tail of 0.2 in
# the rows where float32 is at its worst too), so the rows are held to it as a whole: their median, their ninth
# decile and their worst.  A wrong key, page or state shows as an error of order one in either type.
TOLERANCE = {"float32": 3e-5, "bfloat16": 3e-2}
BF16_NINTH_DECILE, BF16_WORST = 0.1, 0.45


class VononexModel:
    def __init__(self, cfg_dict, seed=0, edit=None, root=None):
        from transformers_neuronx_b200.config import config_from_dict
        from transformers_neuronx_b200.models.decoder import DecoderModel
        from transformers_neuronx_b200.weights import save_safetensors, random_tensors
        self.cfg_dict = copy.deepcopy(cfg_dict)
        arch, self.cfg = config_from_dict(self.cfg_dict)
        self._tmp = tempfile.TemporaryDirectory(prefix="tnx_vononex_", dir=root)
        self.folder = self._tmp.name
        specs = DecoderModel(arch.build_spec(self.cfg)).tensor_specs()
        tensors = random_tensors(specs, seed, self.cfg.init_std, torch.bfloat16)
        tensors = {k: v.to(torch.bfloat16) for k, v in tensors.items()}      # every tensor is stored in bfloat16
        if edit is not None:
            edit(tensors)
        self.cfg.save(self.folder)
        save_safetensors(tensors, os.path.join(self.folder, "model.safetensors"), metadata={"format": "pt"})
        from safetensors.torch import load_file            # the plain side reads the file with another reader
        self.plain_tensors = load_file(os.path.join(self.folder, "model.safetensors"))
        self._cache = {}

    def plain_logits(self, ids):
        key = tuple(int(i) for i in ids)
        if key not in self._cache:
            self._cache[key] = VP.forward_logits(key, self.plain_tensors, self.cfg_dict).float()
        return self._cache[key]

    def random_ids(self, n, seed):
        g = torch.Generator().manual_seed(seed)
        return torch.randint(0, self.cfg.vocab, (n,), generator=g).tolist()


def compare(model: VononexModel, requests, steps, results, dtype, tol=None):
    """Every wanted row against the plain logits of its request at its position, as a fraction of the largest
    plain logit of that row; returns the worst."""
    tol = TOLERANCE[dtype] if tol is None else tol
    pos = {rid: 0 for rid in requests}
    worst, errs = 0.0, []
    for s in steps:
        row = 0
        for e in s["entries"]:
            rid, n = e["id"], len(e["tokens"])
            assert list(e["tokens"]) == list(requests[rid][pos[rid]:pos[rid] + n]), "trace builder bug"
            for w in e.get("want", []):
                got = torch.from_numpy(results[s["step"]][row].copy())
                want = model.plain_logits(requests[rid])[pos[rid] + w]
                err = float((got - want).abs().max()) / float(want.abs().max())
                worst = max(worst, err)
                errs.append(err)
                assert err <= (tol if dtype == "float32" else BF16_WORST), (f"{dtype} step {s['step']} request {rid} position {pos[rid] + w} "
                                    f"({'decoded' if n == 1 else 'portion of %d' % n}): relative error {err:.3e} > {tol:.1e}")
                row += 1
            pos[rid] += n
    if dtype != "float32" and errs:
        errs.sort()
        assert errs[len(errs) // 2] <= tol, f"{dtype}: median relative error {errs[len(errs) // 2]:.3e} > {tol:.1e}"
        assert errs[(len(errs) * 9) // 10] <= BF16_NINTH_DECILE, f"{dtype}: ninth decile {errs[(len(errs) * 9) // 10]:.3e}"
    return worst


def whole_steps(reqs):
    return [{"step": i, "entries": [{"id": rid, "tokens": ids, "want": list(range(len(ids)))}], "end": [rid]}
            for i, (rid, ids) in enumerate(reqs.items())]


def cut_steps(reqs, sizes, tail=0):
    """Each request alone: portions of the given sizes in turn (its last `tail` tokens one by one); every
    position's logits are wanted."""
    steps, k = [], 0
    for rid, ids in reqs.items():
        at = 0
        while at < len(ids):
            n = 1 if len(ids) - at <= tail else min(sizes[k % len(sizes)], len(ids) - tail - at if tail else len(ids) - at)
            n = max(n, 1)
            k += 1
            steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": ids[at:at + n], "want": list(range(n))}],
                          "end": [rid] if at + n == len(ids) else []})
            at += n
    return steps


def mixed_steps(reqs, sizes, max_live=4, decode_tail=6):
    """Up to max_live live requests a step: portions of prompts beside single tokens; a request's last
    decode_tail tokens come one by one; a finished request's place is taken by the next one."""
    waiting = list(reqs)
    live, at, steps, k = [], {r: 0 for r in reqs}, [], 0
    while waiting or live:
        while waiting and len(live) < max_live:
            live.append(waiting.pop(0))
        entries, end = [], []
        for rid in list(live):
            ids = reqs[rid]
            left_ = len(ids) - at[rid]
            n = 1 if left_ <= decode_tail else min(sizes[k % len(sizes)], left_ - decode_tail)
            k += 1
            if k % 7 == 3 and len(live) > 1:
                continue                                   # a request may be left out of a step
            entries.append({"id": rid, "tokens": ids[at[rid]:at[rid] + n], "want": sorted({0, n - 1})})
            at[rid] += n
            if at[rid] == len(ids):
                end.append(rid)
                live.remove(rid)
        if entries:
            steps.append({"step": len(steps), "entries": entries, "end": end})
    return steps
