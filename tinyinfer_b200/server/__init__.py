"""Client side of the batching server: wire protocol, launcher helper and the load generator."""
from pathlib import Path

from .. import LIB_DIR


def binary() -> Path:
    path = LIB_DIR / "tinyinfer_server"
    if not path.exists():
        raise FileNotFoundError(f"{path} is not built; run `python -m tinyinfer_b200.build`")
    return path
