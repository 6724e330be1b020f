import json
import os

import numpy as np
import pytest
import torch

from crosslayer_coding_b200.activation_generation.synthetic import SyntheticSpec, write_synthetic_dataset
from crosslayer_coding_b200.io import hdf5, manifest
from crosslayer_coding_b200.training.data import ChunkRowSampler, LocalActivationStore


# ------------------------------------------------------------------------------------------ HDF5
@pytest.mark.parametrize("dtype", ["bfloat16", "float16", "float32"])
@pytest.mark.parametrize("compression,chunk_rows", [(None, None), ("gzip", 16), (None, 0)])
def test_hdf5_roundtrip_including_negative_bf16(tmp_path, dtype, compression, chunk_rows):
    torch.manual_seed(0)
    layers = {}
    raw = {}
    for l in (0, 1, 2, 10, 20, 100):
        x, y = torch.randn(50, 8), -torch.rand(50, 8) - 0.5  # targets are all negative
        raw[l] = (x, y)
        layers[l] = (hdf5.to_storage_array(x, dtype), hdf5.to_storage_array(y, dtype))
    path = str(tmp_path / "chunk_0.hdf5")
    hdf5.write_chunk_file(path, layers, compression=compression, chunk_rows=chunk_rows)
    with hdf5.H5File(path) as f:
        assert f.layer_groups() == ["layer_0", "layer_1", "layer_2", "layer_10", "layer_20", "layer_100"]  # numeric order
        ds = f["layer_100/targets"]
        assert ds.shape == (50, 8)
        back = hdf5.from_storage_array(ds.read_all(), dtype).float()
        tol = {"bfloat16": 1e-2, "float16": 1e-3, "float32": 0}[dtype]
        assert torch.allclose(back, raw[100][1], atol=tol, rtol=tol)
        assert (back < 0).all()  # negative bf16 values survive (bit patterns, no value conversion)
        rows = [49, 0, 17, 17, 3]
        assert np.array_equal(ds.read_rows(rows), layers[100][1][rows])
        assert np.array_equal(f["layer_2/inputs"][5:9], layers[2][0][5:9])
        with pytest.raises(OSError):
            ds.read_rows([50])
        assert "layer_2/inputs" in f and "layer_3/inputs" not in f


def test_hdf5_many_chunks_two_level_index(tmp_path):
    x = np.arange(200 * 4, dtype=np.float32).reshape(200, 4)
    path = str(tmp_path / "c.h5")
    with hdf5.H5Writer(path) as w:
        w.add("layer_0", "inputs", x, chunk_rows=2)  # 100 chunks > 64 per B-tree node
        w.add("layer_0", "targets", x, chunk_rows=2, gzip_level=1)
    with hdf5.H5File(path) as f:
        assert np.array_equal(f["layer_0/inputs"].read_all(), x)
        assert np.array_equal(f["layer_0/targets"].read_rows([199, 1, 64]), x[[199, 1, 64]])


def test_h5py_cross_check_when_available(tmp_path):
    h5py = pytest.importorskip("h5py")
    x = np.random.rand(40, 6).astype(np.float32)
    p = str(tmp_path / "ours.h5")
    with hdf5.H5Writer(p) as w:
        w.add("layer_0", "inputs", x, chunk_rows=16, gzip_level=4)
    with h5py.File(p, "r") as f:
        assert np.array_equal(f["layer_0/inputs"][:], x)
    p2 = str(tmp_path / "theirs.h5")
    with h5py.File(p2, "w") as f:
        f.create_group("layer_0").create_dataset("inputs", data=x, chunks=(16, 6), compression="gzip")
    with hdf5.H5File(p2) as f:
        assert np.array_equal(f["layer_0/inputs"].read_all(), x)


def test_not_an_hdf5_file(tmp_path):
    p = tmp_path / "junk.h5"
    p.write_bytes(b"x" * 4096)
    with pytest.raises(OSError):
        hdf5.H5File(str(p))


# ------------------------------------------------------------------------------------------ manifest
def test_manifest_both_layouts(tmp_path):
    p3 = str(tmp_path / "a.bin")
    manifest.write_index_3field(p3, [(0, 100, 0), (1, 60, 100)])
    assert os.path.getsize(p3) == 32
    assert manifest.read_index(p3, 160) == {0: 100, 1: 60}
    pairs = np.array([[c, r] for c, n in ((0, 6), (1, 4)) for r in range(n)], dtype=np.uint32)
    p2 = str(tmp_path / "b.bin")
    manifest.write_index_legacy(p2, pairs)
    assert manifest.read_index(p2, 10) == {0: 6, 1: 4}
    # a 16-byte-multiple legacy file whose "token counts" do not add up falls back to the legacy layout
    pairs2 = np.array([[0, r] for r in range(8)], dtype=np.uint32)
    manifest.write_index_legacy(p2, pairs2)
    assert manifest.read_index(p2, 8) == {0: 8}
    with pytest.raises(ValueError):
        manifest.parse_index_bytes(b"12345")


# ------------------------------------------------------------------------------------------ sampler
def _all_rows(s):
    seen = []
    for b in s:
        assert b.shape == (s.batch, 2) and b.dtype == np.uint32
        seen.extend((int(c), int(r)) for c, r in b)
    return seen


@pytest.mark.parametrize("strategy", ["sequential", "random_chunk"])
def test_sampler_completeness_and_sharding(strategy):
    sizes = {0: 32, 1: 32}
    rows = [_all_rows(ChunkRowSampler(sizes, 2, 8, 0, 0, r, 2, strategy, True)) for r in range(2)]
    assert len(rows[0]) == len(rows[1]) == 32
    assert not set(rows[0]) & set(rows[1])
    assert set(rows[0]) | set(rows[1]) == {(c, r) for c in sizes for r in range(32)}
    unsharded = _all_rows(ChunkRowSampler(sizes, 2, 8, 0, 0, 0, 2, strategy, False))
    assert len(set(unsharded)) == 64


def test_sampler_drops_chunk_tails_and_epoch_determinism():
    s = ChunkRowSampler({0: 20, 1: 9}, 2, 8, 1, 0, 0, 1)
    assert len(s) == 3 and len(_all_rows(s)) == 24
    a = _all_rows(ChunkRowSampler({0: 20, 1: 9}, 2, 8, 1, 0, 0, 1))
    b = _all_rows(ChunkRowSampler({0: 20, 1: 9}, 2, 8, 1, 0, 0, 1))
    c = _all_rows(ChunkRowSampler({0: 20, 1: 9}, 2, 8, 1, 1, 0, 1))
    assert a == b and a != c


@pytest.mark.parametrize("strategy", ["sequential", "random_chunk"])
def test_sampler_state_dict_resumes_exactly(strategy):
    mk = lambda: ChunkRowSampler({0: 40, 1: 40, 2: 24}, 3, 8, 5, 0, 0, 1, strategy)  # noqa: E731
    ref = mk()
    for _ in range(4):
        next(ref)
    state = json.loads(json.dumps(ref.state_dict()))  # state must be JSON-serialisable and small
    rest = [next(ref) for _ in range(5)]
    res = mk()
    res.load_state_dict(state)
    for want in rest:
        assert np.array_equal(next(res), want)


# ------------------------------------------------------------------------------------------ local store
@pytest.fixture()
def dataset(tmp_path):
    spec = SyntheticSpec(num_layers=3, d_model=8, dict_size=16, active_mean=3, seed=4)
    return write_synthetic_dataset(str(tmp_path / "ds"), spec, total_tokens=96, chunk_tokens=32, dtype="bfloat16")


def _read_raw(dataset):
    out = {}
    for cid in range(3):
        with hdf5.open_chunk(dataset, cid) as f:
            for l in range(3):
                out[(cid, l)] = (hdf5.from_storage_array(f[f"layer_{l}/inputs"].read_all()).float(),
                                 hdf5.from_storage_array(f[f"layer_{l}/targets"].read_all()).float())
    return out


def test_local_store_batches_match_files_in_sampler_order(dataset):
    st = LocalActivationStore(dataset, train_batch_size_tokens=16, device="cpu", dtype="float32", normalization_method="none",
                              seed=3, prefetch_batches=2)
    raw = _read_raw(dataset)
    twin = ChunkRowSampler(st.chunk_sizes, st.num_chunks, 16, 3, 0, 0, 1)
    n = 0
    for (x, y), idx in zip(st, twin):
        n += 1
        for l in range(3):
            want_x = torch.stack([raw[(int(c), l)][0][int(r)] for c, r in idx])
            want_y = torch.stack([raw[(int(c), l)][1][int(r)] for c, r in idx])
            assert torch.equal(x[l], want_x) and torch.equal(y[l], want_y)
        assert x.stacked.shape == (3, 16, 8)
    assert n == len(st) == 6
    st.close()


def test_local_store_mean_std_normalisation(dataset):
    st = LocalActivationStore(dataset, train_batch_size_tokens=32, device="cpu", dtype="float32", normalization_method="auto")
    stats = manifest.load_norm_stats(dataset)
    raw = _read_raw(dataset)
    allx = torch.cat([raw[(c, 1)][0] for c in range(3)])
    mean = torch.tensor(stats["1"]["inputs"]["mean"])
    std = torch.tensor(stats["1"]["inputs"]["std"])
    got = torch.cat([x[1] for x, _ in st])
    want = (allx - mean) / (std + 1e-6)
    assert torch.allclose(got.sort(dim=0).values, want.sort(dim=0).values, atol=1e-5)
    assert torch.allclose(st.std_tg[2].flatten(), torch.tensor(stats["2"]["targets"]["std"]) + 1e-6)
    st.close()


def test_local_store_state_dict_resume_and_epoch_advance(dataset):
    mk = lambda: LocalActivationStore(dataset, train_batch_size_tokens=16, device="cpu", dtype="float32", seed=9)  # noqa: E731
    a = mk()
    for _ in range(2):
        next(a)
    state = a.state_dict()
    rest = [next(a)[0].stacked.clone() for _ in range(3)]
    b = mk()
    b.load_state_dict(state)
    for want in rest:
        assert torch.equal(next(b)[0].stacked, want)
    for _ in range(1):
        next(b)
    with pytest.raises(StopIteration):
        next(b)
    b.advance_epoch()
    assert next(b)[0].stacked.shape == (3, 16, 8)
    a.close()
    b.close()


def test_local_store_truncated_chunk_raises_after_retries(dataset, monkeypatch):
    import crosslayer_coding_b200.training.data.manifest_activation_store as mod

    monkeypatch.setattr(mod.time, "sleep", lambda s: None)
    # cut every chunk file short: the row data of the later datasets lies outside the file
    for cid in range(3):
        path = os.path.join(dataset, f"chunk_{cid}.hdf5")
        size = os.path.getsize(path)
        with open(path, "r+b") as f:
            f.truncate(size // 2)
    st = LocalActivationStore(dataset, train_batch_size_tokens=16, device="cpu", dtype="float32")
    opened = {"n": 0}
    orig = st._open

    def counting(cid):
        opened["n"] += 1
        return orig(cid)

    st._open = counting
    with pytest.raises(RuntimeError):
        for _ in range(3):  # first failing batch is skipped, the second one ends the stream
            next(st)
    assert opened["n"] >= 6  # three attempts per failing batch
    st.close()


def test_row_sharded_assembly_fills_only_this_ranks_rows(dataset):
    """Tensor-parallel staging assembles 1/W of a batch per rank: the union over the ranks equals the full batch."""
    full = LocalActivationStore(dataset, train_batch_size_tokens=16, device="cpu", dtype="float32", seed=3, shard_data=False)
    idx = next(full.sampler)
    want = torch.zeros(2, 3, 16, 8, dtype=full._storage_torch)
    full._assemble(idx, want)
    got = torch.zeros_like(want)
    for r in range(4):
        part = LocalActivationStore(dataset, train_batch_size_tokens=16, device="cpu", dtype="float32", seed=3, shard_data=False)
        part.row_shard = (4 * r, 4)
        buf = torch.full_like(want, 7)  # rows of other ranks must stay untouched
        part._assemble(idx, buf)
        assert torch.equal(buf[:, :, 4 * r:4 * r + 4], want[:, :, 4 * r:4 * r + 4])
        untouched = torch.ones(16, dtype=torch.bool)
        untouched[4 * r:4 * r + 4] = False
        assert (buf[:, :, untouched].float() == 7).all()
        got[:, :, 4 * r:4 * r + 4] = buf[:, :, 4 * r:4 * r + 4]
        part.close()
    assert torch.equal(got, want)
    full.close()


def test_stager_options_are_inert_on_cpu():
    """The staging options of tensor-parallel GPU runs (targets stay with the token owners, copies gated on an event of the
    consumer's step) must not change anything on a CPU stager."""
    import torch

    from crosslayer_coding_b200.training.data.staging import DeviceStager

    st = DeviceStager((2, 2, 8, 4), torch.float32, torch.device("cpu"), depth=3)
    assert st.push_only_leading(2) is False and st.gate is None
    st.gate = lambda: None
    slot, host = st.host_slot()
    host.copy_(torch.arange(128, dtype=torch.float32).view(2, 2, 8, 4))
    st.submit(slot)
    got = st.acquire(slot)
    assert torch.equal(got, host)
    st.release(slot)
