"""Server settings from the environment (reference: clt_server/core/config.py:5-27).

``STORAGE_BASE_DIR`` (default ``./server_data``), ``CHUNK_RETRY_ATTEMPTS``, ``LOG_LEVEL``; a ``.env`` file in the
working directory is honoured for the same keys.  No pydantic-settings dependency.
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from pathlib import Path


def _dotenv(path: str = ".env") -> dict:
    out = {}
    try:
        with open(path, encoding="utf-8") as fh:
            for line in fh:
                line = line.strip()
                if line and not line.startswith("#") and "=" in line:
                    k, v = line.split("=", 1)
                    out[k.strip()] = v.strip().strip('"').strip("'")
    except OSError:
        pass
    return out


@dataclass
class Settings:
    STORAGE_BASE_DIR: Path = Path("./server_data")
    CHUNK_RETRY_ATTEMPTS: int = 3
    LOG_LEVEL: str = "info"

    @classmethod
    def from_env(cls) -> "Settings":
        env = {**_dotenv(), **os.environ}
        s = cls(
            STORAGE_BASE_DIR=Path(env.get("STORAGE_BASE_DIR", "./server_data")),
            CHUNK_RETRY_ATTEMPTS=int(env.get("CHUNK_RETRY_ATTEMPTS", 3)),
            LOG_LEVEL=env.get("LOG_LEVEL", "info"),
        )
        s.STORAGE_BASE_DIR.mkdir(parents=True, exist_ok=True)
        return s


settings = Settings.from_env()
