"""Per-shape launch autotuner of the tuned kernels.

Replaces the reference's ``benchmarks/benchmark_block_sizes.py`` (a sweep over CUDA thread
block shapes): here the knobs are the kernels' launch *variants* — tile height / width,
lattice rows and column segments per thread of the TMA forward, voxels per thread and
resident blocks of the fused 2D backward, unsplit or role-split consumer warps of the 3D
backward.  For a given problem shape the tuner times every
variant of every (kernel family, dilation) on synthetic data with CUDA events, installs
the winners in the library's launch table (``msd_tuning_set``) and remembers them in a JSON
cache keyed by GPU name and shape, so that later processes only look them up.

    from msd_pytorch_b200 import autotune
    autotune.tune(batch=8, spatial=(512, 512), channels=50, dilations=range(1, 11))

The cache file is ``$MSD_B200_TUNE_CACHE`` or ``~/.cache/msd_pytorch_b200/tuning.json``.
"""
import json
import os

import torch

from . import _lib
from . import msd_custom_convolutions as cc

FAMILIES_2D = {"forward": _lib.FAMILY_FWD2D, "backward": _lib.FAMILY_BWD2D}
FAMILIES_3D = {"forward": _lib.FAMILY_FWD3D, "backward": _lib.FAMILY_BWD3D}


def cache_path():
    return os.environ.get("MSD_B200_TUNE_CACHE") or os.path.join(os.path.expanduser("~"), ".cache", "msd_pytorch_b200", "tuning.json")


def _load_cache():
    try:
        with open(cache_path()) as f:
            return json.load(f)
    except Exception:
        return {}


def _save_cache(cache):
    path = cache_path()
    try:
        os.makedirs(os.path.dirname(path), exist_ok=True)
        tmp = path + ".tmp%d" % os.getpid()
        with open(tmp, "w") as f:
            json.dump(cache, f, indent=1, sort_keys=True)
        os.replace(tmp, path)
    except OSError:
        pass  # a read-only home only costs the re-tuning next time


def shape_key(device, batch, spatial, channels):
    name = torch.cuda.get_device_name(device)
    return "%s|B%d|%s|C%d" % (name, batch, "x".join(str(int(s)) for s in spatial), channels)


def _time(fn, reps):
    for _ in range(2):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / reps


def apply(choices):
    """Install ``{family_name: {dilation: variant}}`` in the library's launch table."""
    for fam, per_d in choices.items():
        code = {"forward2d": _lib.FAMILY_FWD2D, "backward2d": _lib.FAMILY_BWD2D, "forward3d": _lib.FAMILY_FWD3D,
                "backward3d": _lib.FAMILY_BWD3D}[fam]
        for d, v in per_d.items():
            _lib.check(_lib.lib.msd_tuning_set(code, int(d), int(v)))


def reset():
    """Back to the library's default variants."""
    for code in (_lib.FAMILY_FWD2D, _lib.FAMILY_BWD2D, _lib.FAMILY_FWD3D, _lib.FAMILY_BWD3D):
        for d in range(0, 33):
            _lib.lib.msd_tuning_set(code, d, -1)


def tune(batch, spatial, channels, dilations, device=None, reps=5, use_cache=True, verbose=False):
    """Time every launch variant for layers of ``channels`` input channels on a
    ``[batch, channels + 1, *spatial]`` float32 buffer and install the fastest per
    (family, dilation).  Returns ``{family_name: {dilation: variant}}``."""
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    nd = len(spatial)
    key = shape_key(device, batch, spatial, channels)
    cache = _load_cache() if use_cache else {}
    dilations = sorted(set(int(d) for d in dilations))
    if key in cache and all(str(d) in cache[key].get("forward%dd" % nd, {}) for d in dilations):
        choices = {fam: {int(d): v for d, v in per_d.items()} for fam, per_d in cache[key].items()}
        apply(choices)
        return choices
    fams = FAMILIES_2D if nd == 2 else FAMILIES_3D
    g = torch.Generator(device=device).manual_seed(0)
    res = torch.rand(batch, channels + 1, *spatial, device=device, generator=g)
    grad = torch.randn(batch, channels + 1, *spatial, device=device, generator=g)
    w = torch.randn(1, channels, *([3] * nd), device=device, generator=g) * 0.05
    b = torch.zeros(1, device=device)
    gw, gb = torch.zeros_like(w), torch.zeros(1, device=device)
    from .msd_block import block_backward_

    choices = {"forward%dd" % nd: {}, "backward%dd" % nd: {}}
    for d in dilations:
        if any(d > s for s in spatial):
            continue
        for name, code in fams.items():
            nvar = _lib.lib.msd_tuning_num_variants(code)
            best, best_t = 0, None
            for v in range(max(nvar, 1)):
                _lib.check(_lib.lib.msd_tuning_set(code, d, v))
                if name == "forward":
                    t = _time(lambda: cc.conv_relu_forward(res[:, :channels], w, b, res[:, channels:channels + 1], d), reps)
                else:
                    t = _time(lambda: block_backward_(res, grad, channels, [d], [w], [gw], gb), reps)
                if verbose:
                    print("autotune %s%dd d=%d variant %d: %.3f ms" % (name, nd, d, v, t))
                if best_t is None or t < best_t:
                    best, best_t = v, t
            _lib.check(_lib.lib.msd_tuning_set(code, d, best))
            choices["%s%dd" % (name, nd)][d] = best
    if _lib.device_status(device) != 0:
        raise RuntimeError("autotune: a kernel reported a bounded-wait time-out")
    if use_cache:
        cache[key] = {fam: {str(d): v for d, v in per_d.items()} for fam, per_d in choices.items()}
        _save_cache(cache)
    return choices
