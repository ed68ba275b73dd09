"""Data readers, transforms, the python dataset path and the data coordinator on CPU."""
import os
import pickle

import numpy as np
import pytest
import torch

import lbann_b200 as lbann
from lbann_b200.data.coordinator import DataCoordinator
from lbann_b200.data.readers import build_reader
from lbann_b200.data.transforms import build_pipeline
from lbann_b200.proto import reader_pb2


def _proto(name, role="train", **kw):
    r = reader_pb2.Reader()
    r.name, r.role, r.shuffle, r.fraction_of_data_to_use = name, role, False, 1.0
    for k, v in kw.items():
        setattr(r, k, v)
    return r


def test_numpy_npz_csv_readers(tmp_path):
    rs = np.random.RandomState(0)
    mat = np.concatenate([rs.randn(10, 5).astype(np.float32), rs.randint(0, 3, (10, 1)).astype(np.float32)], 1)
    np.save(tmp_path / "m.npy", mat)
    r = build_reader(_proto("numpy", data_filedir=str(tmp_path), data_filename="m.npy", num_labels=3))
    r.setup(0)
    assert r.num_samples() == 10 and r.dims("samples") == (5,) and r.dims("labels") == (3,)
    np.testing.assert_allclose(r.fetch_field("samples", 4), mat[4, :5])
    assert r.fetch_field("labels", 4).argmax() == int(mat[4, 5])

    np.savez(tmp_path / "z.npz", data=rs.randn(6, 2, 3).astype(np.float32), responses=rs.randn(6, 2).astype(np.float32))
    z = build_reader(_proto("numpy_npz", data_filedir=str(tmp_path), data_filename="z.npz"))
    z.setup(0)
    assert z.dims("samples") == (2, 3) and z.dims("responses") == (2,)

    np.savetxt(tmp_path / "c.csv", mat, delimiter=",", header="a,b,c,d,e,y", comments="")
    c = build_reader(_proto("csv", data_filedir=str(tmp_path), data_filename="c.csv", has_header=True,
                            num_labels=3, label_col=5))
    c.setup(0)
    assert c.num_samples() == 10 and c.dims("samples") == (5,)
    np.testing.assert_allclose(c.fetch_field("samples", 2), mat[2, :5], rtol=1e-5)


class _Squares(lbann.util.data.Dataset):
    def __len__(self):
        return 12

    def __getitem__(self, i):
        return lbann.util.data.Sample(sample=np.full((2, 2), float(i), np.float32), response=np.array([i * i], np.float32))

    def get_sample_dims(self):
        return lbann.util.data.SampleDims(sample=[2, 2], response=[1])


def test_python_dataset_reader_round_trip(tmp_path):
    path = str(tmp_path / "ds.pkl")
    msg = lbann.util.data.construct_python_dataset_reader(_Squares(), path, "train", shuffle=False)
    msg.python_dataset.module_dir = os.path.dirname(os.path.abspath(__file__))
    r = build_reader(msg)
    r.setup(0)
    assert r.num_samples() == 12 and r.dims("samples") == (2, 2)
    assert float(r.fetch_field("responses", 5)[0]) == 25.0


def test_transform_pipeline_normalize_and_crop():
    """Image transforms work on height x width x channel images until ``to_lbann_layout``
    turns them channel-major; ``normalize`` then acts per channel."""
    t1, t2, t3 = reader_pb2.Transform(), reader_pb2.Transform(), reader_pb2.Transform()
    t1.center_crop.height, t1.center_crop.width = 4, 4
    t2.to_lbann_layout.SetInParent()
    t3.normalize.means, t3.normalize.stddevs = "1 2 3", "2 2 2"
    pipe = build_pipeline([t1, t2, t3])
    img = np.arange(6 * 6 * 3, dtype=np.float32).reshape(6, 6, 3)
    out = pipe(img.copy())
    chw = img[1:5, 1:5].transpose(2, 0, 1) / 255.0       # the layout step maps bytes to [0, 1]
    want = (chw - np.array([1, 2, 3], np.float32)[:, None, None]) / 2
    assert out.shape == (3, 4, 4)
    np.testing.assert_allclose(out, want, rtol=1e-5, atol=1e-6)


def test_coordinator_deals_every_sample_once_per_epoch_across_ranks():
    seen = []
    for rank in range(2):
        r = build_reader(_proto("synthetic", num_samples=20, synth_dimensions="3"))
        r.setup(1)
        dc = DataCoordinator({"train": r}, 8, dp_rank=rank, dp_size=2, seed=1, background=False)
        dc.start_epoch("training")
        while True:
            b = dc.next_batch("training")
            if b is None:
                break
            seen += list(b.indices)
            assert b.global_size in (8, 4)
            if b.end_of_epoch:
                break
        dc.shutdown()
    assert sorted(seen) == list(range(20))
