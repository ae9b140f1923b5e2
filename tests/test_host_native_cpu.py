"""Host-side C++ helpers: the batched sample gather and the blending index against their Python forms, their error
codes, and a run of all of them under AddressSanitizer + UndefinedBehaviorSanitizer in a child process."""
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from linear_moe_b200.data import datasets as D
from linear_moe_b200.utils import hostlib


def _corpus(tmp_path, dtype=np.uint16, n_docs=37, seed=0):
    rng = np.random.RandomState(seed)
    docs = [rng.randint(0, 60000 if dtype != np.uint8 else 255, size=rng.randint(1, 90)).astype(dtype) for _ in range(n_docs)]
    prefix = str(tmp_path / f"corpus_{np.dtype(dtype).name}")
    D.IndexedDataset.write(prefix, docs, dtype=dtype)
    return prefix


@pytest.mark.parametrize("dtype", [np.uint16, np.int32, np.uint8, np.int64])
def test_native_gather_matches_per_sample_walk(tmp_path, dtype):
    lib = hostlib.load()
    if lib is None:
        pytest.skip("host library not built")
    ds = D.GPTDataset(D.IndexedDataset(_corpus(tmp_path, dtype)), seq_length=32, num_samples=120, seed=7)
    idx = list(range(0, len(ds), 3)) + [len(ds) + 5, 0, 0]
    got = ds.__getitems__(idx)
    assert len(got) == len(idx)
    for i, g in zip(idx, got):
        want = ds[i]["text"]
        assert g["text"].dtype == torch.int64 and g["text"].shape == (33,) and torch.equal(g["text"], want)
    # through a DataLoader the batched fetch is what runs
    dl = torch.utils.data.DataLoader(ds, batch_size=8, shuffle=False)
    first = next(iter(dl))["text"]
    assert torch.equal(first, torch.stack([ds[i]["text"] for i in range(8)]))


def test_native_gather_reports_bad_tables(tmp_path):
    lib = hostlib.load()
    if lib is None:
        pytest.skip("host library not built")
    ds = D.GPTDataset(D.IndexedDataset(_corpus(tmp_path)), seq_length=16, num_samples=40)
    args = dict(lib=lib, data=ds.ds.data, dtype_code=ds.ds.dtype_code, sizes=ds._sizes, pointers=ds._pointers,
                doc_idx=ds.doc_idx, sample_idx=ds.sample_idx, indices=np.array([0, 1]), seq_length=16)
    assert hostlib.gather_gpt_samples(**args).shape == (2, 17)
    with pytest.raises(ValueError, match="outside its table"):
        hostlib.gather_gpt_samples(**{**args, "indices": np.array([len(ds.sample_idx) - 1])})
    with pytest.raises(ValueError, match="outside its table"):
        hostlib.gather_gpt_samples(**{**args, "doc_idx": ds.doc_idx + 1000})
    with pytest.raises(ValueError, match="outside the .bin file"):
        hostlib.gather_gpt_samples(**{**args, "pointers": ds._pointers + ds.ds.data.nbytes})
    with pytest.raises(ValueError, match="seq_length"):
        hostlib.gather_gpt_samples(**{**args, "seq_length": 15})
    with pytest.raises(ValueError, match="integer type"):
        hostlib.gather_gpt_samples(**{**args, "dtype_code": 7})


def test_native_blending_matches_python(monkeypatch):
    lib = hostlib.load()
    if lib is None:
        pytest.skip("host library not built")
    sets = [list(range(1000)) for _ in range(3)]
    a = D.BlendedDataset(sets, [0.5, 0.3, 0.2], 500)
    monkeypatch.setattr(hostlib, "_LIB", None)
    monkeypatch.setattr(hostlib, "_TRIED", True)
    b = D.BlendedDataset(sets, [0.5, 0.3, 0.2], 500)
    assert np.array_equal(a.ds_index, b.ds_index) and np.array_equal(a.ds_sample, b.ds_sample)
    counts = np.bincount(a.ds_index, minlength=3) / 500
    assert np.allclose(counts, [0.5, 0.3, 0.2], atol=0.01)
    with pytest.raises(ValueError, match="1 to 256"):
        D.BlendedDataset([[0]] * 257, [1.0] * 257, 4)


_CHILD = r"""
import sys, numpy as np
from linear_moe_b200.data import datasets as D
from linear_moe_b200.utils import hostlib
lib = hostlib.load()
assert lib is not None and hostlib.lib_path().endswith("_asan.so")
rng = np.random.RandomState(1)
docs = [rng.randint(0, 60000, size=rng.randint(1, 50)).astype(np.uint16) for _ in range(64)]
prefix = sys.argv[1] + "/c"
D.IndexedDataset.write(prefix, docs, dtype=np.uint16)
ds = D.GPTDataset(D.IndexedDataset(prefix), seq_length=24, num_samples=90)
rows = ds.__getitems__(list(range(len(ds))))
for i in (0, 5, len(ds) - 1):
    assert (rows[i]["text"].numpy() == ds[i]["text"].numpy()).all()
for bad in (dict(indices=np.array([10 ** 9])), dict(seq_length=23), dict(pointers=ds._pointers + 10 ** 9)):
    kw = dict(lib=lib, data=ds.ds.data, dtype_code=ds.ds.dtype_code, sizes=ds._sizes, pointers=ds._pointers,
              doc_idx=ds.doc_idx, sample_idx=ds.sample_idx, indices=np.arange(4), seq_length=24)
    kw.update(bad)
    try:
        hostlib.gather_gpt_samples(**kw)
        raise SystemExit("no error for " + str(list(bad)))
    except ValueError:
        pass
b = D.BlendedDataset([list(range(100))] * 4, [0.4, 0.3, 0.2, 0.1], 300)
assert len(b) == 300
print("SANITIZED_OK")
"""


def test_host_helpers_under_asan_ubsan(tmp_path):
    """The same calls in a child process that loads the sanitizer build of the library (ASan runtime preloaded): any
    out-of-bounds access, misaligned load or signed overflow in the helpers aborts the child."""
    from linear_moe_b200 import build
    runtime = subprocess.run(["g++", "-print-file-name=libasan.so"], capture_output=True, text=True).stdout.strip()
    if not runtime or not os.path.isabs(runtime) or not os.path.exists(runtime):
        pytest.skip("no AddressSanitizer runtime beside the compiler")
    so = build.build_host(sanitize=True, out_dir=str(tmp_path))
    env = dict(os.environ, LMOE_HOST_LIB=so, LD_PRELOAD=runtime, ASAN_OPTIONS="detect_leaks=0:abort_on_error=1",
               UBSAN_OPTIONS="halt_on_error=1:print_stacktrace=1")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env["PYTHONPATH"] = root + os.pathsep + env.get("PYTHONPATH", "")
    r = subprocess.run([sys.executable, "-c", _CHILD, str(tmp_path)], env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "SANITIZED_OK" in r.stdout, (r.stdout[-2000:], r.stderr[-4000:])


def test_blended_dataset_batched_fetch(tmp_path):
    a = D.GPTDataset(D.IndexedDataset(_corpus(tmp_path, np.uint16, seed=1)), seq_length=16, num_samples=60, seed=3)
    b = D.GPTDataset(D.IndexedDataset(_corpus(tmp_path, np.int32, seed=2)), seq_length=16, num_samples=60, seed=4)
    blend = D.BlendedDataset([a, b], [0.7, 0.3], 50)
    idx = [0, 7, 3, 49, 12, 12, 51]
    got = blend.__getitems__(idx)
    for i, g in zip(idx, got):
        assert torch.equal(g["text"], blend[i % 50]["text"])
    from linear_moe_b200.dist.mesh import single_process_mesh
    it = D.BatchIterator(blend, 4, single_process_mesh(), torch.device("cpu"))
    first = next(it)
    assert first["tokens"].shape == (4, 16)
    assert torch.equal(first["tokens"], torch.stack([blend[i]["text"][:-1] for i in range(4)]))


def test_prefetching_iterator_keeps_the_order_and_masks_after_eod(tmp_path):
    """--num-workers: the read-ahead thread delivers the same micro-batches in the same order, a resume position discards
    what was read ahead; --eod-mask-loss removes the loss where the input token is the end-of-document id."""
    from linear_moe_b200.dist.mesh import single_process_mesh
    ds = D.GPTDataset(D.IndexedDataset(_corpus(tmp_path, np.uint16, seed=5)), seq_length=16, num_samples=80, seed=9)
    mesh, dev = single_process_mesh(), torch.device("cpu")
    plain = D.BatchIterator(ds, 3, mesh, dev)
    ahead = D.BatchIterator(ds, 3, mesh, dev, prefetch=2)
    for _ in range(7):
        a, b = next(plain), next(ahead)
        assert all(torch.equal(a[k], b[k]) for k in a)
    assert ahead.consumed == plain.consumed == 21
    ahead.consumed = plain.consumed = 6                       # resume elsewhere
    a, b = next(plain), next(ahead)
    assert torch.equal(a["tokens"], b["tokens"]) and torch.equal(a["tokens"][0], ds[6]["text"][:-1])
    ahead._shutdown()
    eod = int(a["tokens"][0, 3])
    masked = next(D.BatchIterator(ds, 3, mesh, dev, consumed_samples=6, eod_token=eod, eod_mask_loss=True))
    assert torch.equal(masked["tokens"], a["tokens"])
    assert bool((masked["loss_mask"][a["tokens"] == eod] == 0).all()) and masked["loss_mask"][0, 3] == 0
    assert bool((masked["loss_mask"][a["tokens"] != eod] == 1).all())

    class Broken(torch.utils.data.Dataset):
        def __len__(self):
            return 4

        def __getitem__(self, i):
            raise OSError("disk gone")
    with pytest.raises(OSError, match="disk gone"):
        next(D.BatchIterator(Broken(), 2, mesh, dev, prefetch=1))


def test_index_cache_is_written_once_and_reused(tmp_path, monkeypatch):
    prefix = _corpus(tmp_path, np.uint16, seed=8)
    cache = tmp_path / "cache"
    a = D.GPTDataset(D.IndexedDataset(prefix), seq_length=16, num_samples=70, seed=2, cache_dir=str(cache))
    files = sorted(os.listdir(cache))
    assert len(files) == 3 and all(f.endswith(".npy") for f in files)
    monkeypatch.setattr(D, "build_sample_idx", lambda *a, **k: (_ for _ in ()).throw(AssertionError("rebuilt")))
    b = D.GPTDataset(D.IndexedDataset(prefix), seq_length=16, num_samples=70, seed=2, cache_dir=str(cache))
    assert all(torch.equal(a[i]["text"], b[i]["text"]) for i in range(0, len(a), 7))
    assert torch.equal(a.__getitems__([1, 2, 3])[2]["text"], b.__getitems__([1, 2, 3])[2]["text"])
    with pytest.raises(AssertionError, match="rebuilt"):          # another seed is another index
        D.GPTDataset(D.IndexedDataset(prefix), seq_length=16, num_samples=70, seed=3, cache_dir=str(cache))
