"""On-disk store of tuned kernel configurations.

The reference keeps tuned configurations only in module dictionaries
(tritonix/ops/matmul.py:267-268), so every process pays the minutes-long first call again.  Here
the winner of ``TunableKernel.tune`` is also written next to the dispatcher's files:
``<cache dir>/tuned/<kernel>.json`` maps ``"m,n,k[,extra]|dtype|device|library version"`` to the
configuration dict.  ``TRITONIX_B200_TUNE_CACHE=0`` disables reading and writing.
"""
from __future__ import annotations

import json
import logging
import os
import tempfile
import threading
from typing import Optional

from tritonix_b200.dispatcher import cache_dir

log = logging.getLogger("tritonix.autotune")
_lock = threading.Lock()


def _enabled() -> bool:
    return os.environ.get("TRITONIX_B200_TUNE_CACHE", "1") not in ("0", "false", "off")


def _path(kernel: str):
    return cache_dir() / "tuned" / f"{kernel}.json"


def make_key(shape_key: tuple, dtype, device_name: str, version: str) -> str:
    return "|".join([",".join(str(x) for x in shape_key), str(dtype), device_name, version])


def load(kernel: str, key: str) -> Optional[dict]:
    if not _enabled():
        return None
    try:
        with open(_path(kernel)) as f:
            cfg = json.load(f).get(key)
        return dict(cfg) if isinstance(cfg, dict) else None
    except FileNotFoundError:
        return None
    except Exception as exc:  # unreadable / corrupted: behave as a miss
        log.debug("tuned-config cache unreadable (%s): %s", kernel, exc)
        return None


def save(kernel: str, key: str, cfg: dict) -> None:
    if not _enabled() or cfg is None:
        return
    path = _path(kernel)
    with _lock:
        try:
            path.parent.mkdir(parents=True, exist_ok=True)
            try:
                with open(path) as f:
                    data = json.load(f)
                if not isinstance(data, dict):
                    data = {}
            except Exception:
                data = {}
            data[key] = cfg
            fd, tmp = tempfile.mkstemp(dir=path.parent, suffix=".tmp")
            with os.fdopen(fd, "w") as f:
                json.dump(data, f, indent=1, sort_keys=True)
            os.replace(tmp, path)
        except Exception as exc:
            log.warning("could not persist the tuned configuration for %s: %s", kernel, exc)
