"""The stand-alone utilities of ``lbann_b200.tools``."""
import gzip
import struct

import numpy as np

from lbann_b200.tools import compute_mean, mnist_to_npy, partition_input_list


def test_partition_input_list(tmp_path):
    src = tmp_path / "list.txt"
    src.write_text("".join(f"dir with space/img{i}.png {i % 7}\n" for i in range(103)))
    base = tmp_path / "out" 
    assert partition_input_list.main([str(src), str(base), "4", "--seed", "3"]) == 0
    whole = partition_input_list.read_list(str(base))
    assert sorted(whole) == sorted(partition_input_list.read_list(str(src))) and len(whole) == 103
    parts = [partition_input_list.read_list(f"{base}.p{p}") for p in range(4)]
    assert all(len(p) == 25 for p in parts)
    flat = [r for p in parts for r in p]
    assert flat == whole[:100]                    # partitions are consecutive runs of the shuffle
    assert len(set(flat)) == 100
    assert whole != partition_input_list.read_list(str(src))


def test_mean_image_and_uniform(tmp_path):
    rng = np.random.default_rng(0)
    root = tmp_path / "imgs"
    root.mkdir()
    names, crops = [], []
    for i in range(5):
        img = rng.integers(0, 255, size=(20 + i, 24 + 2 * i, 3), dtype=np.uint8)
        np.save(root / f"a{i}.npy", img)
        names.append(f"a{i}.npy")
        y0, x0 = (img.shape[0] - 16) // 2, (img.shape[1] - 12) // 2
        crops.append(img[y0:y0 + 16, x0:x0 + 12].astype(np.float64))
    (tmp_path / "list.txt").write_text("".join(f"{n} 0\n" for n in names))
    out = tmp_path / "out"
    assert compute_mean.main(["compute", str(root), str(tmp_path / "list.txt"), str(out),
                              "--crop", "12", "16", "--save-cropped"]) == 0
    mean = np.load(out / "mean.npy")
    np.testing.assert_allclose(mean, np.mean(crops, 0), rtol=1e-6)
    assert np.array_equal(np.load(out / "cropped" / "a3.npy"), crops[3].astype(np.uint8))
    # two emulated ranks add up to the same mean
    parts = []
    for r in range(2):
        total = np.zeros((16, 12, 3))
        n = 0
        for i in range(r, 5, 2):
            total += crops[i]
            n += 1
        parts.append((total, n))
    np.testing.assert_allclose((parts[0][0] + parts[1][0]) / (parts[0][1] + parts[1][1]), mean, rtol=1e-6)
    assert compute_mean.main(["uniform", str(tmp_path / "u.npy"), "--size", "4", "3",
                              "--values", "1", "2", "3"]) == 0
    u = np.load(tmp_path / "u.npy")
    assert u.shape == (3, 4, 3) and np.all(u[:, :, 1] == 2)
    assert compute_mean.main(["uniform", str(tmp_path / "v.npy"), "--from-image", str(out / "mean.npy")]) == 0
    v = np.load(tmp_path / "v.npy")
    np.testing.assert_allclose(v[0, 0], mean.reshape(-1, 3).mean(0), rtol=1e-5)


def test_mnist_idx_conversion(tmp_path):
    rng = np.random.default_rng(1)
    src = tmp_path / "raw"
    src.mkdir()
    for stem, n in (("train", 9), ("t10k", 4)):
        imgs = rng.integers(0, 255, size=(n, 28, 28), dtype=np.uint8)
        labs = rng.integers(0, 10, size=(n,), dtype=np.uint8)
        with gzip.open(src / f"{stem}-images-idx3-ubyte.gz", "wb") as f:
            f.write(struct.pack(">HBBIII", 0, 8, 3, n, 28, 28) + imgs.tobytes())
        with open(src / f"{stem}-labels-idx1-ubyte", "wb") as f:
            f.write(struct.pack(">HBBI", 0, 8, 1, n) + labs.tobytes())
        if stem == "train":
            keep = (imgs, labs)
    assert mnist_to_npy.main([str(src), str(tmp_path / "out")]) == 0
    comb = np.load(tmp_path / "out" / "train.npy")
    assert comb.shape == (9, 785)
    assert np.array_equal(comb[:, :784], keep[0].reshape(9, -1)) and np.array_equal(comb[:, 784], keep[1])
    z = np.load(tmp_path / "out" / "test.npz")
    assert z["data"].shape == (4, 784) and z["labels"].shape == (4,)


def test_viz_writes_a_dot_graph_with_subgrid_colours(tmp_path):
    import lbann_b200 as lbann
    from lbann_b200.tools import viz
    x = lbann.Input(data_field="samples", name="in")
    a = lbann.FullyConnected(x, num_neurons=4, name="left", grid_tag=1)
    b = lbann.FullyConnected(x, num_neurons=4, name="right", grid_tag=2)
    y = lbann.Sum([a, b], name="join")
    model = lbann.Model(1, layers=list(lbann.traverse_layer_graph(x)))
    lbann.proto.serialize.save_prototext(str(tmp_path / "m.prototext"), trainer=lbann.Trainer(mini_batch_size=2),
                                         model=model, data_reader=None, optimizer=lbann.SGD(learn_rate=0.1))
    assert viz.main([str(tmp_path / "m.prototext"), str(tmp_path / "g.dot"), "--label-format", "type-and-name",
                     "--color-cross-grid"]) == 0
    dot = open(tmp_path / "g.dot").read()
    assert dot.startswith("digraph model {") and '"in" -> "left" [color="red"' in dot
    assert '"left" [label="fully_connected\\nleft", fillcolor="#a0c4ff"]' in dot
    assert '"right" -> "join"' in dot and y is not None


def test_print_times_reads_the_statistics_lines(tmp_path, capsys):
    from lbann_b200.tools import print_times
    log = """\
some other output
model0 (instance 0) training epoch 0 objective function : 2.30412
model0 (instance 0) training epoch 0 accuracy : 11.5%
model0 (instance 0) training epoch 0 run time : 3.25s
model0 (instance 0) training epoch 0 mini-batch time statistics : 0.0125s mean, 0.012s median, 0.02s max, 0.011s min, 0.001s stdev
model0 (instance 0) validation objective function : 2.1
model0 (instance 0) training epoch 1 objective function : 1.5
"""
    (tmp_path / "run.log").write_text(log)
    rows = print_times.parse(log.splitlines())
    assert ("model0", "training", 0, "accuracy", 11.5) in rows and ("model0", "validation", -1, "objective function", 2.1) in rows
    assert print_times.main([str(tmp_path / "run.log"), "--csv", str(tmp_path / "t.csv")]) == 0
    out = capsys.readouterr().out.splitlines()
    assert out[0].split()[:3] == ["model", "mode", "epoch"] and "mini-batch time statistics" in out[0]
    csv_rows = open(tmp_path / "t.csv").read().splitlines()
    assert csv_rows[1].startswith("model0,training,0,2.30412,11.5,3.25,0.0125")


def test_every_command_line_option_of_the_reference_is_accepted():
    """Option names are the reference's (src/utils/options.cpp); a command line written for it
    parses here, including the switches that have no counterpart."""
    from lbann_b200.utils import options as opts
    o = opts.reset()
    rest = o.parse(["--omp_num_threads=8", "--init_nvshmem", "--checkpoint_dir", "ck", "--num_lists=3",
                    "--trainer_enable_subgrid_async_comm", "--data_store_test_cache", "--not_an_option"])
    assert rest == ["--not_an_option"]
    assert o.get_int("omp_num_threads") == 8 and o.get_bool("init_nvshmem") and o.get("checkpoint_dir") == "ck"
    assert o.get_int("num_lists") == 3 and o.get_bool("trainer_enable_subgrid_async_comm")
    assert o.get("smiles_buffer_size") == 16 * 1024 * 1024 and not o.get_bool("caliper")
    assert "--omp_num_threads" in o.describe()
    opts.reset()
