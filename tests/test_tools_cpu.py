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
