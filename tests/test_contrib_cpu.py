"""lbann.contrib: site tables and launch defaults, experimental modules against numpy."""
import math

import numpy as np
import pytest
import torch

import lbann_b200 as lbann
from lbann_b200.contrib import systems


def test_site_detection_and_machine_tables():
    assert systems.detect({}, "lassen708.llnl.gov") == ("lc", "lassen")
    assert systems.detect({"NERSC_HOST": "perlmutter"}, "nid001234") == ("nersc", "perlmutter")
    assert systems.detect({"LMOD_SYSTEM_NAME": "frontier"}, "login01") == ("olcf", "frontier")
    assert systems.detect({}, "my-workstation") == (None, None)
    assert systems.params("lc", "lassen") == systems.System(44, 4, "lsf")
    assert systems.procs_per_node("lc", "quartz") == 2          # CPU machine: one process per socket
    assert systems.procs_per_node("olcf", "frontier") == 8
    with pytest.raises(RuntimeError, match="unknown lc system"):
        systems.params("lc", "nosuchmachine")
    from lbann_b200.contrib.lc import systems as lc
    assert lc.gpus_per_node("tioga") == 8 and lc.scheduler("tioga") == "flux" and lc.has_gpu("pascal")
    from lbann_b200.contrib.riken import systems as riken
    assert riken.scheduler("fugaku") == "pjm" and not riken.has_gpu("fugaku")
    from lbann_b200.contrib.lc import paths
    assert paths.imagenet_labels("lassen", "val", 100).endswith("labels/val_c0-99.txt")
    assert paths.mnist_dir("lassen").startswith("/p/gpfs1/")


def test_site_launcher_fills_scheduler_processes_and_environment(tmp_path):
    from lbann_b200.contrib import launcher
    kw = launcher.site_defaults("lc", "lassen", {"nodes": 2})
    assert kw["scheduler"] == "lsf" and kw["procs_per_node"] == 4 and kw["nodes"] == 2
    assert kw["environment"]["OMP_NUM_THREADS"] == "10"          # 44 cores / 4 processes - 1
    kw = launcher.site_defaults("olcf", "frontier", {"procs_per_node": 4, "environment": {"NCCL_SOCKET_IFNAME": "x"}})
    assert kw["procs_per_node"] == 4 and kw["environment"]["NCCL_SOCKET_IFNAME"] == "x"
    script = launcher.site_make_batch_script("lc", system="corona", work_dir=str(tmp_path), nodes=1)
    assert type(script).__name__ == "FluxBatchScript"
    from lbann_b200.contrib.nersc import launcher as nersc
    script = nersc.make_batch_script(system="perlmutter", work_dir=str(tmp_path), nodes=1)
    assert type(script).__name__ == "SlurmBatchScript"


def _evaluate(layers_fn, feed):
    """Run a layer graph on one mini-batch and return the outputs of the returned layers."""
    x = lbann.Input(data_field="samples")
    outs = layers_fn(x)
    outs = outs if isinstance(outs, (list, tuple)) else [outs]
    names = []
    for i, l in enumerate(outs):
        l.name = l.name or f"out{i}"
        names.append(l.name)
    res = lbann.evaluate(lbann.Model(1, layers=list(lbann.traverse_layer_graph([x] + list(outs)))), feed, names)
    res = res if isinstance(res, tuple) else (res,)
    return [np.asarray(r) for r in res]


def test_fftshift_matches_numpy():
    from lbann_b200.contrib.modules import FFTShift
    rng = np.random.RandomState(0)
    for dims in ((2, 5, 6), (1, 4, 3, 5)):
        data = rng.rand(3, *dims).astype(np.float32)
        out, inv = _evaluate(lambda x: [FFTShift()(lbann.Reshape(x, dims=list(dims)), dims),
                                        FFTShift(inverse=True)(lbann.Reshape(x, dims=list(dims)), dims)],
                             data.reshape(3, -1))
        axes = tuple(range(2, data.ndim))
        np.testing.assert_array_equal(out.reshape(data.shape), np.fft.fftshift(data, axes=axes))
        np.testing.assert_array_equal(inv.reshape(data.shape), np.fft.ifftshift(data, axes=axes))


def test_radial_profile_matches_binned_means():
    from lbann_b200.contrib.modules import RadialProfile
    rng = np.random.RandomState(1)
    dims, max_r = (2, 7, 6), 4
    data = rng.rand(3, *dims).astype(np.float32)
    (out,) = _evaluate(lambda x: RadialProfile()(lbann.Reshape(x, dims=list(dims)), dims, max_r), data.reshape(3, -1))
    r, counts = RadialProfile.radial_bins(dims[1:], max_r)
    want = np.zeros((3, dims[0], max_r), dtype=np.float64)
    for b in range(max_r):
        if counts[b]:
            want[:, :, b] = data[:, :, r == b].mean(axis=-1)
    np.testing.assert_allclose(out.reshape(want.shape), want, rtol=1e-5, atol=1e-6)


def test_contrib_objective_functions():
    from lbann_b200.contrib.modules import objective_functions as of
    rng = np.random.RandomState(2)
    p = rng.rand(4, 6).astype(np.float32) * 0.8 + 0.1
    k = rng.randint(0, 5, (4, 6)).astype(np.float32)
    feed = np.concatenate([p, k], axis=1)

    def graph(x):
        sl = lbann.Slice(x, axis=0, slice_points=[0, 6, 12])
        pred, lab = lbann.Identity(sl), lbann.Identity(sl)
        return [of.GeometricDistributionNegativeLogLikelihood()([pred, lab]),
                of.PoissonDistributionNegativeLogLikelihood()([pred, lab]),
                of.CrossEntropyWithUncertainty()([pred, lbann.Clamp(lab, min=0.0, max=1.0)])]
    geo, poi, ceu = _evaluate(graph, feed)
    np.testing.assert_allclose(geo.reshape(-1), -(k * np.log(1 - p) + np.log(p)).sum(1), rtol=1e-5)
    lgam = np.vectorize(math.lgamma)(k + 1)
    np.testing.assert_allclose(poi.reshape(-1), (p - k * np.log(p) + lgam).sum(1), rtol=2e-3)
    np.testing.assert_allclose(ceu.reshape(-1), -np.log((p * np.clip(k, 0, 1)).sum(1)), rtol=1e-5)


def test_group_lasso_and_l1_of_a_weights_matrix():
    from lbann_b200.contrib.modules import objective_functions as of
    vals = np.arange(1, 13, dtype=np.float32).reshape(3, 4) - 6.0      # width 3 (rows here), height 4
    w = lbann.Weights(initializer=lbann.ValueInitializer(values=[float(v) for v in vals.reshape(-1)]),
                      optimizer=lbann.NoOptimizer(), name="lasso_w")
    gl, l1 = _evaluate(lambda x: [of.GroupLasso(w, 4, 3)(), of.L1WeightRegularization(w, [3, 4])()],
                       np.zeros((2, 1), dtype=np.float32))
    np.testing.assert_allclose(gl.reshape(-1)[0], np.sqrt((vals ** 2).sum(1)).sum(), rtol=1e-5)
    np.testing.assert_allclose(l1.reshape(-1)[0], np.abs(vals).sum(), rtol=1e-6)


def test_wide_resnet_doubles_the_inner_widths_only():
    from lbann_b200.contrib.models import WideResNet50_2
    from lbann_b200.models import ResNet50
    x = lbann.Input(data_field="samples")
    wide = WideResNet50_2(10)(x)
    convs = [l for l in lbann.traverse_layer_graph(x) if type(l).__name__ == "Convolution"]
    by_name = {l.name: l for l in convs}
    a = next(l for n, l in by_name.items() if "layer1_block0_branch2a" in n)
    b = next(l for n, l in by_name.items() if "layer1_block0_branch2b" in n)
    c = next(l for n, l in by_name.items() if "layer1_block0_branch2c" in n)
    assert (a.out_channels, b.out_channels, c.out_channels) == (128, 128, 256)
    y = lbann.Input(data_field="samples")
    ResNet50(10)(y)
    narrow = next(l for l in lbann.traverse_layer_graph(y)
                  if type(l).__name__ == "Convolution" and "layer1_block0_branch2b" in l.name)
    assert narrow.out_channels == 64 and wide is not None


def test_single_tensor_reader_functions(tmp_path, monkeypatch):
    import importlib
    data = np.arange(12, dtype=np.float32).reshape(4, 3)
    np.save(tmp_path / "data.npy", data)
    monkeypatch.setenv("LBANN_SINGLE_TENSOR_FILE", str(tmp_path / "data.npy"))
    mod = importlib.reload(importlib.import_module("lbann_b200.contrib.single_tensor_data_reader"))
    assert mod.num_samples() == 4 and mod.sample_dims() == (3,)
    np.testing.assert_array_equal(mod.get_sample(2), data[2])


def test_smiles_tokenizer_and_masked_molecule_dataset(tmp_path):
    from lbann_b200.contrib.data.chem_tokenizers import ChemTokenizer, ChemTokenType, SMILESTokenizer, TOKENIZERS
    from lbann_b200.contrib.data.molecule_dataset import ChemTextDataset, IGNORE, TextDatasetWithOffsets
    mols = ["CC(=O)Oc1ccccc1C(=O)O", "zinc42|C[C@H](N)C(=O)O", "BrCCCl", "[Na+].[Cl-]", "C%12CC%12"]
    tok = SMILESTokenizer(vocab=ChemTokenizer.build_vocab(mols, SMILESTokenizer(vocab=list(
        ("[PAD]", "[UNK]", "[CLS]", "[SEP]", "[MASK]"))).tokenize))
    assert tok.tokenize(mols[2]) == ["Br", "C", "C", "Cl"]                       # two-letter elements stay whole
    assert tok.tokenize(mols[1])[:2] == ["C", "[C@H]"]                           # name before "|" dropped, bracket atom whole
    assert tok.tokenize(mols[4]) == ["C", "%12", "C", "C", "%12"]
    ids = tok.encode(mols[3], max_length=12)
    assert len(ids) == 12 and ids[0] == tok.cls_token_id and ids.count(tok.pad_token_id) == 12 - 5
    assert tok.decode(ids) == "[Na+].[Cl-]"
    assert tok.encode("CSC")[2] == tok.unk_token_id                                  # an element the vocabulary lacks
    with pytest.raises(ModuleNotFoundError):
        TOKENIZERS[ChemTokenType.SELFIES]("x")
    vocab_file, data_file = tmp_path / "vocab.txt", tmp_path / "mols.txt"
    vocab_file.write_text("\n".join(tok.ids_to_tokens[i] for i in range(len(tok))) + "\n")
    data_file.write_text("\n".join(mols) + "\n")
    assert TextDatasetWithOffsets.write_offsets(str(data_file)) == 5
    for offsets in (False, True):
        ds = ChemTextDataset(str(data_file), str(vocab_file), seqlen=16, mlm_probability=0.5, attn_mask=True,
                             use_offsets=offsets, seed=3)
        assert len(ds) == 5 and ds.get_sample_dims().sample == [48]
        s = ds[0].sample
        inp, lab, att = s[:16].astype(int), s[16:32].astype(int), s[32:].astype(int)
        clean = np.asarray(tok.encode(mols[0], max_length=16))
        picked = lab != IGNORE
        assert picked.any() and (lab[picked] == clean[picked]).all()
        assert (inp[~picked] == clean[~picked]).all()                            # untouched positions keep their ids
        assert not picked[0] and att.tolist() == (clean != tok.pad_token_id).astype(int).tolist()
        np.testing.assert_array_equal(ds[0].sample, s)                           # deterministic per (seed, index)
    import pickle
    assert pickle.loads(pickle.dumps(ds))[1].sample.shape == (48,)


def test_reference_import_paths_resolve():
    """Module paths of the reference's Python package that scripts import directly."""
    import importlib
    for name in ("launcher.slurm", "launcher.lsf", "launcher.flux", "launcher.pjm", "launcher.openmpi",
                 "models.alexnet", "modules.attention_allsubgraph", "modules.pytorch", "modules.graph.dense",
                 "modules.graph.sparse", "modules.graph.utils", "proto.text2bin", "proto.bin2text",
                 "torch.converters", "torch.helpers", "torch.lowering", "torch.opaque", "contrib.data.chem_tokenizers",
                 "contrib.data.molecule_dataset", "contrib.lc.launcher", "contrib.nersc.systems"):
        importlib.import_module("lbann_b200." + name)
    from lbann_b200.modules.pytorch import PytorchLinear, PytorchMatmul
    x = lbann.Input(data_field="samples")
    y, shape = PytorchLinear(lbann.Reshape(x, dims=[2, 3, 4]), (2, 3, 4), 5, return_dims=True)
    assert shape == (2, 3, 5)
    (out,) = _evaluate(lambda inp: PytorchMatmul(lbann.Reshape(inp, dims=[2, 2, 3, 2]), (2, 2, 3, 2),
                                                 lbann.Reshape(lbann.Slice(inp, axis=0, slice_points=[0, 16]),
                                                               dims=[2, 2, 2, 2]), (2, 2, 2, 2)),
                       np.arange(2 * 24, dtype=np.float32).reshape(2, 24))
    a = np.arange(48, dtype=np.float32).reshape(2, 2, 2, 3, 2)
    b = a.reshape(2, 24)[:, :16].reshape(2, 2, 2, 2, 2)
    np.testing.assert_allclose(out.reshape(2, 2, 2, 3, 2), a @ b, rtol=1e-6)


def test_prototext_binary_round_trip_tools(tmp_path):
    from lbann_b200.proto.bin2text import bin2text
    from lbann_b200.proto.text2bin import text2bin
    x = lbann.Input(data_field="samples")
    y = lbann.FullyConnected(x, num_neurons=3, name="fc")
    model = lbann.Model(1, layers=list(lbann.traverse_layer_graph(x)))
    lbann.proto.serialize.save_prototext(str(tmp_path / "a.prototext"), trainer=lbann.Trainer(mini_batch_size=2),
                                         model=model, data_reader=None, optimizer=lbann.SGD(learn_rate=0.1))
    text2bin(str(tmp_path / "a.prototext"), str(tmp_path / "a.protobin"))
    bin2text(str(tmp_path / "a.protobin"), str(tmp_path / "b.prototext"))
    from google.protobuf import text_format
    from lbann_b200.proto import lbann_pb2
    m1, m2 = lbann_pb2.LbannPB(), lbann_pb2.LbannPB()
    text_format.Parse(open(tmp_path / "a.prototext").read(), m1)
    text_format.Parse(open(tmp_path / "b.prototext").read(), m2)
    assert m1 == m2 and m1.model.layer[1].name == "fc" and y is not None
