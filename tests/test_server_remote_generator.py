import json
import os

import numpy as np
import pytest
import torch

from crosslayer_coding_b200.activation_generation.generator import ActivationGenerator, _RunningStat, upload_file_with_retries
from crosslayer_coding_b200.activation_generation.synthetic import SyntheticSpec, write_synthetic_dataset
from crosslayer_coding_b200.config import ActivationConfig
from crosslayer_coding_b200.io import hdf5, manifest
from crosslayer_coding_b200.server import create_app
from crosslayer_coding_b200.training.data import LocalActivationStore, RemoteActivationStore

fastapi_testclient = pytest.importorskip("fastapi.testclient")


class _Bridge:
    """Routes ``requests.get/post`` of the remote store / uploader into the ASGI app (no sockets)."""

    def __init__(self, client, base="http://testserver"):
        self.client, self.base = client, base
        self.fail_next = []  # status codes to return before passing requests through

    def _path(self, url):
        assert url.startswith(self.base), url
        return url[len(self.base):]

    @staticmethod
    def _wrap(resp):
        if not hasattr(resp, "ok"):  # httpx responses lack the requests-style flag
            try:
                resp.ok = resp.status_code < 400
            except AttributeError:
                pass
        return resp

    def get(self, url, **kw):
        kw.pop("timeout", None)
        return self._wrap(self.client.get(self._path(url), **kw))

    def post(self, url, **kw):
        kw.pop("timeout", None)
        if self.fail_next:
            code = self.fail_next.pop(0)

            class R:
                ok = False
                status_code = code
                text = "injected"

                def raise_for_status(self):
                    import requests

                    raise requests.HTTPError(f"{code}")

            return R()
        return self._wrap(self.client.post(self._path(url), **kw))


@pytest.fixture()
def served(tmp_path, monkeypatch):
    src = write_synthetic_dataset(str(tmp_path / "src"), SyntheticSpec(num_layers=2, d_model=8, dict_size=16, active_mean=3, seed=2),
                                  total_tokens=96, chunk_tokens=48, dtype="float16")
    client = fastapi_testclient.TestClient(create_app(str(tmp_path / "root")))
    did = "org/model/ds_train"
    for i in range(2):
        with open(os.path.join(src, f"chunk_{i}.hdf5"), "rb") as fh:
            assert client.post(f"/datasets/{did}/chunks/{i}", files={"chunk_file": (f"chunk_{i}.h5", fh, "application/x-hdf5")}).status_code == 201
    with open(os.path.join(src, "index.bin"), "rb") as fh:
        assert client.post(f"/datasets/{did}/manifest", files={"manifest_file": ("index.bin", fh, "application/octet-stream")}).status_code == 201
    assert client.post(f"/datasets/{did}/metadata", json=json.load(open(os.path.join(src, "metadata.json")))).status_code == 201
    assert client.post(f"/datasets/{did}/norm_stats", json=json.load(open(os.path.join(src, "norm_stats.json")))).status_code == 201
    bridge = _Bridge(client)
    import requests

    monkeypatch.setattr(requests, "get", bridge.get)
    monkeypatch.setattr(requests, "post", bridge.post)
    return src, client, did, bridge


def test_server_routes_and_slice_layout(served):
    src, client, did, _ = served
    assert client.get("/api/v1/health").json() == {"status": "ok"}
    assert client.get(f"/datasets/{did}/info").json()["total_tokens"] == 96
    assert len(client.get(f"/datasets/{did}/manifest").content) == 32
    assert client.get("/datasets/nope/info").status_code == 404
    r = client.post(f"/datasets/{did}/slice?chunk=1", json={"rows": [7, 2, 40]})
    assert r.status_code == 200
    got = np.frombuffer(r.content, dtype=np.float16).reshape(2, 2, 3, 8)  # layer, (inputs|targets), rows, d
    with hdf5.open_chunk(src, 1) as f:
        for l in range(2):
            assert np.array_equal(got[l, 0], f[f"layer_{l}/inputs"].read_rows([2, 7, 40]))  # rows come back sorted
            assert np.array_equal(got[l, 1], f[f"layer_{l}/targets"].read_rows([2, 7, 40]))
    assert client.post(f"/datasets/{did}/slice?chunk=9", json={"rows": [1]}).status_code == 404
    assert client.post(f"/datasets/{did}/slice?chunk=0", json={"rows": []}).status_code == 400
    assert client.post(f"/datasets/{did}/slice?chunk=0", json={"rows": [4800]}).status_code == 400


def test_remote_store_equals_local_store(served):
    src, _, did, _ = served
    kw = dict(train_batch_size_tokens=16, device="cpu", dtype="float32", normalization_method="mean_std", seed=5)
    local = LocalActivationStore(src, **kw)
    remote = RemoteActivationStore("http://testserver", did, **kw)
    assert remote.chunk_sizes == local.chunk_sizes  # the 3-field manifest is understood over HTTP as well
    n = 0
    for (lx, ly), (rx, ry) in zip(local, remote):
        assert torch.equal(lx.stacked, rx.stacked) and torch.equal(ly.stacked, ry.stacked)
        n += 1
    assert n == 6
    local.close()
    remote.close()


def test_remote_store_retries_slice_fetch(served, monkeypatch):
    src, _, did, bridge = served
    import crosslayer_coding_b200.training.data.manifest_activation_store as mod

    monkeypatch.setattr(mod.time, "sleep", lambda s: None)
    remote = RemoteActivationStore("http://testserver", did, train_batch_size_tokens=16, device="cpu", dtype="float32")
    bridge.fail_next = [503, 500]  # two failures, third attempt succeeds
    x, _ = next(remote)
    assert x.stacked.shape == (2, 16, 8)
    remote.close()


def test_uploader_retry_classes(tmp_path):
    cfg = ActivationConfig(model_name="m", mlp_input_module_path_template="a.{}", mlp_output_module_path_template="b.{}",
                           dataset_path="d", upload_max_retries=4, upload_initial_backoff=0.0)
    f = tmp_path / "chunk_0.hdf5"
    f.write_bytes(b"abc")

    class Sess:
        def __init__(self, codes):
            self.codes, self.calls = list(codes), 0

        def post(self, url, **kw):
            self.calls += 1
            code = self.codes.pop(0)

            class R:
                ok = code < 300
                status_code = code
                text = ""

            return R()

    s = Sess([503, 429, 201])
    assert upload_file_with_retries(s, "u", f, "chunk_file", cfg, "x", sleep=lambda t: None) and s.calls == 3
    s = Sess([404, 201])
    assert not upload_file_with_retries(s, "u", f, "chunk_file", cfg, "x", sleep=lambda t: None) and s.calls == 1
    s = Sess([507, 201])
    assert not upload_file_with_retries(s, "u", f, "chunk_file", cfg, "x", sleep=lambda t: None) and s.calls == 1
    s = Sess([500] * 4)
    assert not upload_file_with_retries(s, "u", f, "chunk_file", cfg, "x", sleep=lambda t: None) and s.calls == 4


# ------------------------------------------------------------------------------------------ generator
class _FakeExtractor:
    """Deterministic arange batches, like the mocked extractor of the reference's generator tests."""

    def __init__(self, n_batches=5, batch=40, d=6, layers=(0, 1), negative=False):
        self.n_batches, self.batch, self.d, self.layers, self.negative = n_batches, batch, d, layers, negative

    def stream_activations(self, **kw):
        for b in range(self.n_batches):
            base = torch.arange(self.batch * self.d, dtype=torch.float32).reshape(self.batch, self.d) + 1000 * b
            if self.negative:
                base = -base
            yield ({l: base + 10000 * l for l in self.layers}, {l: base + 10000 * l + 0.5 for l in self.layers})


def _gen_cfg(tmp_path, **kw):
    base = dict(model_name="fake/model", mlp_input_module_path_template="a.{}", mlp_output_module_path_template="b.{}",
                dataset_path="some/dataset", activation_dir=str(tmp_path / "acts"), chunk_token_threshold=80,
                activation_dtype="float32", compression=None)
    base.update(kw)
    return ActivationConfig(**base)


@pytest.mark.parametrize("fmt", ["hdf5", "npz"])
def test_generator_chunks_manifest_metadata_stats(tmp_path, fmt):
    cfg = _gen_cfg(tmp_path, output_format=fmt)
    gen = ActivationGenerator(cfg, device="cpu", extractor=_FakeExtractor())
    gen.generate_and_save()
    out = gen.out_dir
    assert str(out).endswith(os.path.join("fake/model", "dataset_train"))
    meta = json.load(open(out / "metadata.json"))
    assert meta["total_tokens"] == 200 and meta["num_layers"] == 2 and meta["d_model"] == 6 and meta["dtype"] == "float32"
    rec = np.fromfile(out / "index.bin", dtype=manifest.REC3)
    assert rec["num_tokens"].tolist() == [80, 80, 40] and rec["offset"].tolist() == [0, 80, 160]
    if fmt == "hdf5":
        perms = []
        for cid in range(2):
            with hdf5.open_chunk(str(out), cid) as f:
                x0, x1 = f["layer_0/inputs"].read_all(), f["layer_1/inputs"].read_all()
                assert np.array_equal(x1 - 10000, x0)  # one permutation shared by all layers of a chunk
                assert np.allclose(f["layer_0/targets"].read_all(), x0 + 0.5)
                perms.append(x0[:, 0].copy())
                assert not np.array_equal(x0[:, 0], np.sort(x0[:, 0]))  # rows are shuffled
        assert not np.array_equal(perms[0] % 1000, perms[1] % 1000)
    else:
        z = np.load(out / "chunk_0.npz")
        assert z["layer_0_inputs"].shape == (80, 6)
    stats = json.load(open(out / "norm_stats.json"))
    allx = torch.cat([b[0][1] for b in _FakeExtractor().stream_activations()])
    assert np.allclose(stats["1"]["inputs"]["mean"], allx.mean(0).numpy(), rtol=1e-6)
    assert np.allclose(stats["1"]["inputs"]["std"], allx.std(0).numpy(), rtol=1e-6)


def test_generator_bf16_negative_values_roundtrip_through_store(tmp_path):
    cfg = _gen_cfg(tmp_path, activation_dtype="bfloat16", chunk_token_threshold=100, compression="gzip")
    gen = ActivationGenerator(cfg, device="cpu", extractor=_FakeExtractor(n_batches=3, batch=50, negative=True))
    gen.generate_and_save()
    st = LocalActivationStore(str(gen.out_dir), train_batch_size_tokens=50, device="cpu", dtype="float32")
    x, _ = next(st)
    assert (x[0] <= 0).all() and float(x[0].min()) < -100  # the sign bit survives write + read
    st.close()


def test_generator_target_total_tokens_and_uploads(tmp_path, served):
    _, client, _, bridge = served
    cfg = _gen_cfg(tmp_path, target_total_tokens=130, remote_server_url="http://testserver", upload_initial_backoff=0.0)
    import requests

    class Sess:
        post = staticmethod(bridge.post)

    import crosslayer_coding_b200.activation_generation.generator as genmod

    orig = requests.Session
    requests.Session = lambda: Sess()  # uploader threads create their own sessions
    try:
        gen = ActivationGenerator(cfg, device="cpu", extractor=_FakeExtractor())
        gen.set_storage_type("remote")
        gen.generate_and_save()
    finally:
        requests.Session = orig
    did = "fake%2Fmodel%2Fdataset_train"
    info = client.get(f"/datasets/{did}/info")
    assert info.status_code == 200 and info.json()["total_tokens"] == 130
    assert client.post(f"/datasets/{did}/slice?chunk=1", json={"rows": [0, 1]}).status_code == 200
    assert client.get(f"/datasets/{did}/norm_stats").status_code == 200


def test_running_stat_matches_direct():
    torch.manual_seed(0)
    parts = [torch.randn(n, 5) * 3 + 7 for n in (10, 1, 33, 64)]
    rs = _RunningStat(5)
    for p in parts:
        rs.update(p)
    mean, std = rs.finalize()
    full = torch.cat(parts).double()
    assert np.allclose(mean, full.mean(0).numpy()) and np.allclose(std, full.std(0).numpy())
