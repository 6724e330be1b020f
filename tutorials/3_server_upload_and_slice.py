#!/usr/bin/env python
"""Tutorials 3 and 4 - the server protocol by hand: upload chunks, manifest, metadata and norm stats, then fetch
a slice of rows and decode the wire format (reference: tutorials/3-*, 4-*; clt_server/api/endpoints).

The application object is driven in-process through FastAPI's test client: same routes, no socket.

    python tutorials/3_server_upload_and_slice.py
"""
import json
import os

import numpy as np
from fastapi.testclient import TestClient

from _common import L, D, dataset, workdir

from crosslayer_coding_b200.server.app import create_app


def main() -> None:
    root = workdir("3")
    data = dataset(os.path.join(root, "activations"))
    client = TestClient(create_app(os.path.join(root, "server_data")))
    did = "synthetic%2Ftoy_train"  # dataset ids contain a slash: URL-encode it
    n_chunks = len([f for f in os.listdir(data) if f.startswith("chunk_")])
    for c in range(n_chunks):
        with open(os.path.join(data, f"chunk_{c}.hdf5"), "rb") as f:
            r = client.post(f"/datasets/{did}/chunks/{c}", files={"chunk_file": (f"chunk_{c}.hdf5", f, "application/x-hdf5")})
            assert r.status_code == 201, r.text
    with open(os.path.join(data, "index.bin"), "rb") as f:
        assert client.post(f"/datasets/{did}/manifest", files={"manifest_file": ("index.bin", f, "application/octet-stream")}).status_code == 201
    assert client.post(f"/datasets/{did}/metadata", json=json.load(open(os.path.join(data, "metadata.json")))).status_code == 201
    assert client.post(f"/datasets/{did}/norm_stats", json=json.load(open(os.path.join(data, "norm_stats.json")))).status_code == 201
    print("info:", client.get(f"/datasets/{did}/info").json())

    rows = [5, 17, 42, 1000]
    r = client.post(f"/datasets/{did}/slice", params={"chunk": 0}, json={"rows": rows})
    assert r.status_code == 200, r.text
    # wire format: for every layer the inputs block then the targets block, each [len(rows), d_model] in the
    # dataset's dtype (float32 here), layers in ascending order
    flat = np.frombuffer(r.content, dtype=np.float32)
    per_layer = flat.reshape(L, 2, len(rows), D)
    print("slice:", per_layer.shape, "first input row of layer 0:", per_layer[0, 0, 0, :4])


if __name__ == "__main__":
    main()
