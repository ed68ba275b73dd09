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


# ---------------------------------------------------------------------------- sample lists / data store
def _write_bundles(tmp_path, files=3, per_file=4):
    names = {}
    for b in range(files):
        arrays = {}
        for s in range(per_file):
            name = f"s{b}_{s}"
            arrays[f"{name}/samples"] = np.full((2, 2), 10 * b + s, dtype=np.float32)
            arrays[f"{name}/responses"] = np.asarray([b - s], dtype=np.float32)
        np.savez(tmp_path / f"bundle{b}.npz", **arrays)
        names[f"bundle{b}.npz"] = [f"s{b}_{s}" for s in range(per_file)]
    return names


def test_sample_list_inclusion_exclusion_striding_and_round_trip(tmp_path):
    from lbann_b200.data.sample_list import SampleList
    _write_bundles(tmp_path)
    inc = (f"MULTI-SAMPLE_INCLUSION\n5 7 3\n{tmp_path}\n"
           "bundle0.npz 2 2 s0_0 s0_3\nbundle1.npz 1 3 s1_2\nbundle2.npz 2 2 s2_1 s2_2\n")
    sl = SampleList.load_from_string(inc)
    assert sl.samples == [("bundle0.npz", "s0_0"), ("bundle0.npz", "s0_3"), ("bundle1.npz", "s1_2"),
                          ("bundle2.npz", "s2_1"), ("bundle2.npz", "s2_2")]
    exc = (f"MULTI-SAMPLE_EXCLUSION\n9 3 3\n{tmp_path}\n"
           "bundle0.npz 3 1 s0_1\nbundle1.npz 4 0\nbundle2.npz 2 2 s2_0 s2_3\n")
    se = SampleList.load_from_string(exc)
    assert len(se) == 9 and ("bundle0.npz", "s0_1") not in se.samples and ("bundle1.npz", "s1_3") in se.samples
    # every second line for rank 1 of 2
    assert SampleList.load_from_string(inc, stride=2, offset=1).files() == ["bundle1.npz"]
    v2 = SampleList.load_from_string(f"MULTI-SAMPLE_INCLUSION_V2\n2 1\n{tmp_path}\nbundle1.npz 2 s1_0 s1_1\n")
    assert [s for _, s in v2.samples] == ["s1_0", "s1_1"]
    single = SampleList.load_from_string(f"SINGLE-SAMPLE\n2\n{tmp_path}\na.npy 3\nb.npy 5\n")
    assert single.samples == [("a.npy", ""), ("b.npy", "")] and single.labels == ["3", "5"]
    # written lists read back the same; partitions cover the list
    se.write(tmp_path / "again.txt")
    assert SampleList.load(str(tmp_path / "again.txt")).samples == se.samples
    parts = se.partition(2)
    assert sorted(parts[0].samples + parts[1].samples) == sorted(se.samples)
    with pytest.raises(ValueError):
        SampleList.load_from_string(f"MULTI-SAMPLE_INCLUSION\n1 0 1\n{tmp_path}\nbundle0.npz 2 0 s0_0\n")


def test_sample_list_reader_and_single_rank_store(tmp_path):
    from lbann_b200.data.readers import build_reader
    from lbann_b200.data.store import DataStore
    _write_bundles(tmp_path)
    (tmp_path / "list.txt").write_text(
        f"MULTI-SAMPLE_INCLUSION\n4 8 2\n{tmp_path}\nbundle0.npz 2 2 s0_1 s0_2\nbundle2.npz 2 2 s2_0 s2_3\n")
    rp = lbann.reader_pb2.Reader(name="npz_bundle", role="train", sample_list=str(tmp_path / "list.txt"),
                                 fraction_of_data_to_use=1.0)
    r = build_reader(rp).setup(0)
    assert r.num_samples() == 4 and r.dims("samples") == (2, 2)
    b = r.fetch_batch([0, 3], ["samples", "responses"])
    assert b["samples"][:, 0, 0].tolist() == [1.0, 23.0] and b["responses"].reshape(-1).tolist() == [-1.0, -1.0]
    store = DataStore(r)
    for _ in range(3):
        got = store.fetch_batch([3, 1, 0, 2], ["samples"])
        assert got["samples"][:, 0, 0].tolist() == [23.0, 2.0, 1.0, 20.0]
    assert store.stats["file_reads"] == 4 and store.stats["cache_hits"] == 8


@pytest.mark.parametrize("mode", ["dynamic", "preload"])
def test_data_store_exchanges_samples_between_two_ranks(tmp_path, mode):
    from test_distconv_cpu import _run
    res = _run(2, ["store", mode], str(tmp_path / "s.json"))
    stats = res["stats"]
    assert all(s["ok"] for s in stats)
    # every sample was read from the reader exactly once over both ranks and three epochs
    assert sum(s["file_reads"] for s in stats) == res["samples"]
    assert sum(s["cached"] for s in stats) == res["samples"]
    assert sum(s["sent"] for s in stats) == sum(s["received"] for s in stats) > 0


def test_trainer_runs_with_the_data_store_option():
    """--use_data_store puts the cache in front of every reader: two epochs read each sample
    once."""
    from lbann_b200.exec.trainer import ExecTrainer
    from lbann_b200.utils import options as opts
    o = opts.reset()
    o.set("disable_cuda", True)
    o.set("use_data_store", True)
    x = lbann.Input(data_field="samples")
    y = lbann.FullyConnected(x, num_neurons=3)
    loss = lbann.MeanSquaredError(y, lbann.Input(data_field="responses"))
    model = lbann.Model(2, layers=list(lbann.traverse_layer_graph([x])),
                        objective_function=lbann.ObjectiveFunction([loss]))
    r = reader_pb2.Reader(name="synthetic", role="train", num_samples=12, synth_dimensions="5",
                          synth_response_dimensions="3", fraction_of_data_to_use=1.0, shuffle=True)
    dr = reader_pb2.DataReader()
    dr.reader.append(r)
    exp = lbann.proto.serialize.build_experiment(trainer=lbann.Trainer(mini_batch_size=4), model=model,
                                                 data_reader=dr, optimizer=lbann.SGD(learn_rate=0.01))
    tr = ExecTrainer(exp)
    m = tr.build_model(exp.model)
    tr.train(m)
    store = tr.data_coordinator.reader("training")
    tr.shutdown()
    opts.reset()
    assert store.stats["file_reads"] == 12 and store.stats["cache_hits"] >= 12


def test_nci_reader_skips_metadata_columns_and_maps_classes(tmp_path):
    lines = ["broken header line"]
    rows = [("a", "b", 0.5, "rs", "e", 1.0, 2.0, 3.0), ("a", "b", 1.5, "xx", "e", 4.0, 5.0, 6.0)]
    lines += [" ".join(str(v) for v in r) for r in rows]
    (tmp_path / "nci.txt").write_text("\n".join(lines) + "\n")
    r = build_reader(_proto("nci", data_filedir=str(tmp_path), data_filename="nci.txt")).setup(0)
    assert r.num_samples() == 2 and r.dims("samples") == (3,)
    b = r.fetch_batch([0, 1], ["samples", "labels", "responses"])
    assert b["samples"].tolist() == [[1.0, 2.0, 3.0], [4.0, 5.0, 6.0]]
    assert b["labels"].tolist() == [[1.0, 0.0], [0.0, 1.0]]            # "rs" -> class 0
    assert b["responses"].reshape(-1).tolist() == [0.5, 1.5]


def test_mesh_reader_channels_target_and_flips(tmp_path):
    h, w, chans = 4, 6, ("Density", "Pressure")
    rng = np.random.RandomState(0)
    ref = {}
    for c in chans + ("mask",):
        os.makedirs(tmp_path / f"{c}16")
        for i in range(3):
            a = rng.rand(h, w).astype(np.float32)
            ref[(c, i)] = a
            a.tofile(tmp_path / f"{c}16" / f"{c}{i:03d}.bin")
    fmt = f"suffix=16 height={h} width={w} index_length=3 channels={','.join(chans)}"
    r = build_reader(_proto("mesh", data_filedir=str(tmp_path), format=fmt)).setup(0)
    assert r.num_samples() == 3 and r.dims("samples") == (2, h, w) and r.dims("responses") == (h, w)
    b = r.fetch_batch([2], ["samples", "responses"])
    np.testing.assert_array_equal(b["samples"][0, 1].numpy(), ref[("Pressure", 2)])
    np.testing.assert_array_equal(b["responses"][0].numpy(), ref[("mask", 2)])
    # flips: the target of a sample is flipped like its channels
    r2 = build_reader(_proto("mesh", data_filedir=str(tmp_path), format=fmt + " flips")).setup(0)
    for _ in range(6):
        b = r2.fetch_batch([1], ["samples", "responses"])
        fh, fv = r2._flips[1]
        want = ref[("mask", 1)][::-1 if fv else 1, ::-1 if fh else 1]
        np.testing.assert_array_equal(b["responses"][0].numpy(), want)
        np.testing.assert_array_equal(b["samples"][0, 0].numpy(), ref[("Density", 1)][::-1 if fv else 1, ::-1 if fh else 1])
    with pytest.raises(ValueError, match="index length"):
        build_reader(_proto("mesh", data_filedir=str(tmp_path),
                            format=f"suffix=16 height={h} width={w} index_length=0")).setup(0)


def test_pilot2_molecular_reader_neighbours_and_scaling(tmp_path):
    frames, mols, beads, nv, hood = 2, 5, 3, 20, 2
    rng = np.random.RandomState(1)
    feats = rng.rand(frames, mols, beads, nv).astype(np.float32) * 100
    nbrs = np.full((frames, mols, 2 * hood), -1, dtype=np.float32)
    nbrs[1, 3] = [3, 0, -1, 4]                       # entry 0 is the molecule itself
    np.savez(tmp_path / "p2.npz", features=feats, neighbors=nbrs)
    r = build_reader(_proto("pilot2_molecular_reader", data_filedir=str(tmp_path), data_filename="p2.npz",
                            num_neighbors=3, max_neighborhood=hood)).setup(0)
    assert r.num_samples() == frames * mols and r.dims("samples") == (4, beads, nv)
    x = r.fetch_batch([1 * mols + 3], ["samples"])["samples"][0].numpy()
    scale = np.ones(nv, dtype=np.float32)
    scale[:3] = 1 / 320.0
    scale[8:] = 1 / 10.0
    np.testing.assert_allclose(x[0], feats[1, 3] * scale, rtol=1e-6)
    np.testing.assert_allclose(x[1], feats[1, 0] * scale, rtol=1e-6)      # neighbour 0 of the same frame
    assert not x[2].any()                                                 # id -1: left at zero
    np.testing.assert_allclose(x[3], feats[1, 4] * scale, rtol=1e-6)


def test_ras_lipid_reader_sequences_and_normalisation(tmp_path):
    rng = np.random.RandomState(2)
    for f, n in (("a.npz", 5), ("b.npz", 4)):
        np.savez(tmp_path / f, density_sig1=rng.rand(n, 13, 13, 14).astype(np.float64),
                 states=rng.randint(0, 3, n).astype(np.float64), bbs=rng.rand(n, 184, 3).astype(np.float32),
                 probs=rng.rand(n, 3))
    table = np.stack([np.full(14, 2.0), np.full(14, -1.0), np.full(14, 0.5), np.full(14, 0.25)], axis=1)
    np.savetxt(tmp_path / "norm.txt", table)
    rp = _proto("ras_lipid", data_filedir=str(tmp_path), data_file_pattern="*.npz", metadata_filename="norm.txt",
                format="seq_len=2")
    r = build_reader(rp).setup(0)
    assert r.num_samples() == 2 + 2                   # whole sequences only: 5 // 2 + 4 // 2
    assert r.dims("samples") == (2, 13, 13, 14) and r.dims("labels") == (3,)
    za = np.load(tmp_path / "a.npz")
    b = r.fetch_batch([1], ["samples", "labels", "bbs"])
    np.testing.assert_allclose(b["samples"][0].numpy(), (za["density_sig1"][2:4] + 1.0) / 3.0, rtol=1e-5, atol=1e-6)
    assert int(b["labels"][0].argmax()) == int(za["states"][3])            # state of the last frame
    np.testing.assert_allclose(b["bbs"][0].numpy(), za["bbs"][2:4], rtol=1e-6)
    rp.format = "seq_len=1 z_score=1"
    rz = build_reader(rp).setup(0)
    assert rz.num_samples() == 9
    x = rz.fetch_batch([0], ["samples"])["samples"][0].numpy()
    np.testing.assert_allclose(x[0], (za["density_sig1"][0] - 0.5) / 0.25, rtol=1e-5, atol=1e-6)


def test_jag_reader_key_selection_slices_and_normalisation(tmp_path):
    rng = np.random.RandomState(3)
    data = {}
    for s in ("run0", "run1", "run2"):
        for k in ("p0", "p1", "p2"):
            data[f"{s}/inputs/{k}"] = rng.rand(1).astype(np.float32)
        for k in ("yield", "tion", "bang"):
            data[f"{s}/scalars/{k}"] = rng.rand(1).astype(np.float32)
        data[f"{s}/images/view0"] = rng.rand(4, 4).astype(np.float32)
    np.savez(tmp_path / "jag0.npz", **data)
    (tmp_path / "list.txt").write_text(f"MULTI-SAMPLE_INCLUSION\n3 0 1\n{tmp_path}\njag0.npz 3 0 run0 run1 run2\n")
    md = lbann.lbann_pb2.DataSetMetaData() if hasattr(lbann, "lbann_pb2") else None
    if md is None:
        from lbann_b200.proto import lbann_pb2
        md = lbann_pb2.DataSetMetaData()
    md.schema.jag_scalar_keys.extend(["tion", "yield"])
    md.schema.jag_input_keys.extend(["p2", "p0"])
    ind = md.schema.independent.add()
    ind.pieces.extend([2, 1])                           # scalars, then images
    dep = md.schema.dependent.add()
    dep.pieces.append(3)                                # inputs
    for scale, bias in ((2.0, 1.0), (3.0, -1.0)):
        q = md.normalization.jag_scalar_normalization_params.add()
        q.scale, q.bias = scale, bias
    rp = _proto("jag_conduit", sample_list=str(tmp_path / "list.txt"))
    r = build_reader(rp, md).setup(0)
    assert r.num_samples() == 3 and r.dims("samples") == (2 + 16,) and r.dims("responses") == (2,)
    assert r.slice_points("independent") == [0, 2, 18] and r.slice_points("dependent") == [0, 2]
    b = r.fetch_batch([1], ["samples", "responses"])
    want = np.concatenate([data["run1/scalars/tion"] * 2.0 + 1.0, data["run1/scalars/yield"] * 3.0 - 1.0,
                           data["run1/images/view0"].reshape(-1)])
    np.testing.assert_allclose(b["samples"][0].numpy(), want, rtol=1e-6)
    np.testing.assert_allclose(b["responses"][0].numpy(),
                               np.concatenate([data["run1/inputs/p2"], data["run1/inputs/p0"]]), rtol=1e-6)
    md.schema.jag_input_keys.append("nope")
    with pytest.raises(ValueError, match="not in the bundles"):
        build_reader(rp, md).setup(0)


def test_generator_banks_streams_and_checkpoint_state():
    """Named generators: the data-sequence and LTFB streams agree across ranks and trainers,
    model / fast / I/O streams differ per rank (I/O also per thread); the state survives a
    round trip; an epoch's visiting order depends on (seed, epoch) only."""
    from lbann_b200.utils.random import GeneratorBanks, data_order
    a, b = GeneratorBanks(), GeneratorBanks()
    a.init(7, rank_in_world=0, rank_in_trainer=0, trainer=0, num_io_threads=2)
    b.init(7, rank_in_world=3, rank_in_trainer=1, trainer=1, num_io_threads=2)
    assert a.data_seq_generator.integers(1 << 30, size=4).tolist() == b.data_seq_generator.integers(1 << 30, size=4).tolist()
    assert a.ltfb_generator.integers(1 << 30, size=4).tolist() == b.ltfb_generator.integers(1 << 30, size=4).tolist()
    assert a.generator.integers(1 << 30, size=4).tolist() != b.generator.integers(1 << 30, size=4).tolist()
    assert a.io_generator(0).integers(1 << 30, size=4).tolist() != a.io_generator(1).integers(1 << 30, size=4).tolist()
    saved = a.dumps()
    want = [a.generator.random(), a.io_generator(1).random(), a.fast_generator.random()]
    c = GeneratorBanks()
    c.loads(saved)
    assert [c.generator.random(), c.io_generator(1).random(), c.fast_generator.random()] == want
    idx = np.arange(20)
    assert data_order(5, idx, 2).tolist() == data_order(5, idx, 2).tolist() != data_order(5, idx, 3).tolist()
    assert sorted(data_order(5, idx, 2).tolist()) == idx.tolist()


def test_data_store_spill_and_warm_restart(tmp_path):
    """A store writes its cache and ownership table to disk; a new store over the same
    reader restores it and serves every sample without touching the reader again.  Through
    the trainer: --data_store_spill=<dir> makes the second run start warm."""
    from lbann_b200.data.store import DataStore
    _write_bundles(tmp_path)
    (tmp_path / "list.txt").write_text(
        f"MULTI-SAMPLE_INCLUSION\n4 8 2\n{tmp_path}\nbundle0.npz 2 2 s0_1 s0_2\nbundle2.npz 2 2 s2_0 s2_3\n")
    rp = lbann.reader_pb2.Reader(name="npz_bundle", role="train", sample_list=str(tmp_path / "list.txt"),
                                 fraction_of_data_to_use=1.0)
    first = DataStore(build_reader(rp).setup(0), preload=True)
    want = first.fetch_batch([0, 1, 2, 3], ["samples", "responses"])
    path = first.spill(str(tmp_path / "spill"))
    assert os.path.exists(path)
    again = DataStore(build_reader(rp).setup(0))
    assert again.load_spilled(str(tmp_path / "spill")) == 4 and again.preloaded
    got = again.fetch_batch([3, 2, 1, 0], ["samples", "responses"])
    assert again.stats["file_reads"] == 0
    torch.testing.assert_close(got["samples"], want["samples"].flip(0))
    other = DataStore(build_reader(rp).setup(0), rank=1, world=2)
    with pytest.raises(FileNotFoundError):
        other.load_spilled(str(tmp_path / "spill"))

    from lbann_b200.exec.trainer import ExecTrainer
    from lbann_b200.utils import options as opts
    x = lbann.Input(data_field="samples")
    y = lbann.FullyConnected(lbann.Reshape(x, dims=[4]), num_neurons=1, has_bias=False, name="fc")
    loss = lbann.MeanSquaredError(y, lbann.Input(data_field="responses"))
    reads = []
    for _ in range(2):
        o = opts.reset()
        o.set("disable_cuda", True)
        o.set("use_data_store", True)
        o.set("data_store_spill", str(tmp_path / "spill2"))
        model = lbann.Model(1, layers=list(lbann.traverse_layer_graph(x)), objective_function=lbann.ObjectiveFunction([loss]))
        dr = lbann.reader_pb2.DataReader()
        dr.reader.append(rp)
        exp = lbann.proto.serialize.build_experiment(trainer=lbann.Trainer(mini_batch_size=2), model=model,
                                                     data_reader=dr, optimizer=lbann.SGD(learn_rate=0.01))
        tr = ExecTrainer(exp)
        m = tr.build_model(exp.model)
        tr.train(m)
        reads.append(tr.data_coordinator.modes["training"].reader.stats["file_reads"])
        tr.shutdown()
    opts.reset()
    assert reads[0] == 4 and reads[1] == 0, reads
