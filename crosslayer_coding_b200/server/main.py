"""``python -m crosslayer_coding_b200.server.main`` — run the activation server with uvicorn
(``HOST`` / ``PORT`` / ``LOG_LEVEL`` / ``STORAGE_BASE_DIR`` from the environment, reference clt_server/main.py:43-51)."""
from __future__ import annotations

import os

from .app import create_app
from .config import settings

app = create_app()

if __name__ == "__main__":
    import uvicorn

    host = os.getenv("HOST", "127.0.0.1")
    port = int(os.getenv("PORT", "8000"))
    print(f"Starting server on {host}:{port}, storage {settings.STORAGE_BASE_DIR}")
    uvicorn.run(app, host=host, port=port, log_level=os.getenv("LOG_LEVEL", "info"))
