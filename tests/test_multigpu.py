"""Multi-GPU tests (one process per GPU over NCCL + this library's peer-memory kernels)."""
import os

import pytest
import torch

from test_distconv_cpu import _run

pytestmark = pytest.mark.gpu

needs2 = pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
ENV = {"LBANN_TEST_DEVICE": "cuda", "NCCL_NVLS_ENABLE": "0"}
# a learning rate at which the small CosmoFlow stays a contraction, so that runs can be compared
# over more than a couple of steps
STABLE = dict(ENV, LBANN_TEST_LR="0.0005")


def test_first_layer_pooling_fusion_in_the_model(tmp_path):
    """The small CosmoFlow on one GPU with the first pooling layer computed inside the
    first convolution's kernel (the default) and with the two separate kernels: same
    losses and weights; the fused run launches fewer kernels."""
    args = ["cosmoflow", "1", "6", "fp16", "32", "8,16,16"]
    fused = _run(1, args, str(tmp_path / "a.json"), STABLE)
    plain = _run(1, args, str(tmp_path / "b.json"), dict(STABLE, LBANN_DISABLE_CONV_POOL_FUSION="1"))
    assert fused["status"] == 0 and plain["status"] == 0
    assert fused["launches"] < plain["launches"], (fused["launches"], plain["launches"])
    for a, b in zip(fused["losses"], plain["losses"]):
        assert abs(a - b) <= 2e-3 * max(1.0, abs(a)), (fused["losses"], plain["losses"])
    for k, v in plain["weight_norms"].items():
        assert abs(v - fused["weight_norms"][k]) <= 1e-3 * max(1.0, abs(v)), k


@needs2
def test_symmetric_memory_collectives(tmp_path):
    n = min(torch.cuda.device_count(), 4)
    res = _run(n, ["comm"], str(tmp_path / "c.json"), ENV)
    assert res["native"] and res["world"] == n
    assert res["all_ranks_ok"], res


@needs2
@pytest.mark.parametrize("width,channels,graph", [("32", "8,16,16", ""), ("64", "16,32,32", ""),
                                                  ("32", "8,16,16", "graph"),
                                                  ("32", "8,16,16,16,16", "")])
def test_distconv_two_gpus_matches_one(tmp_path, width, channels, graph):
    """Depth split over two GPUs with the halo exchange inside the convolution kernels
    (generic implicit-GEMM kernel at width 32, halo-slab kernel at width 64; eager launches
    and graph replay; five blocks at width 32 leave the last convolution ONE plane per rank,
    as eight ranks do on a 128^3 volume): same losses and weights as one GPU, no interior copies (every
    producer wrote straight into its consumer's tensor with halo planes), clean status."""
    steps = "8" if graph else "5"
    tail = [width, channels] + ([graph] if graph else [])
    single = _run(1, ["cosmoflow", "1", steps, "fp16"] + tail, str(tmp_path / "a.json"), STABLE)
    dist = _run(2, ["cosmoflow", "2", steps, "fp16"] + tail, str(tmp_path / "b.json"), STABLE)
    assert dist["status"] == 0 and dist["sharded_update"]
    assert dist["halo_tensors"] >= 4 and dist["halo_bytes"] > 0
    assert dist["interior_copies"] == 0, dist
    if graph:
        assert dist["graph"]
    for a, b in zip(single["losses"], dist["losses"]):
        assert abs(a - b) <= 1e-2 * max(1.0, abs(a)), (single["losses"], dist["losses"])
    for k, v in single["weight_norms"].items():
        assert abs(v - dist["weight_norms"][k]) <= 5e-3 * max(1.0, abs(v)), k


@needs2
def test_distconv_shuffle_to_sample_parallel_on_gpus(tmp_path):
    """An 8^3 volume on two GPUs: the last pooling would see one plane per rank, so the
    tensor is redistributed to sample-parallel in front of it (one all-to-all kernel each
    way) and the rest of the network runs data-parallel; same results as one GPU."""
    single = _run(1, ["cosmoflow", "1", "4", "fp16", "8"], str(tmp_path / "a.json"), STABLE)
    dist = _run(2, ["cosmoflow", "2", "4", "fp16", "8"], str(tmp_path / "b.json"), STABLE)
    assert dist["status"] == 0
    for a, b in zip(single["losses"], dist["losses"]):
        assert abs(a - b) <= 1e-2 * max(1.0, abs(a)), (single["losses"], dist["losses"])
    for k, v in single["weight_norms"].items():
        assert abs(v - dist["weight_norms"][k]) <= 5e-3 * max(1.0, abs(v)), k


@needs2
def test_sharded_update_matches_replicated(tmp_path):
    """Reduce-scatter -> update of the owned blocks -> peer stores of the new values gives
    the same trajectory as all-reduce -> the same update on every rank."""
    a = _run(2, ["cosmoflow", "2", "5", "fp16"], str(tmp_path / "a.json"), STABLE)
    b = _run(2, ["cosmoflow", "2", "5", "fp16"], str(tmp_path / "b.json"),
             dict(STABLE, LBANN_REPLICATED_OPTIMIZER="1"))
    assert a["sharded_update"] and not b["sharded_update"]
    for x, y in zip(a["losses"], b["losses"]):
        assert abs(x - y) <= 1e-3 * max(1.0, abs(x)), (a["losses"], b["losses"])
    for k, v in a["weight_norms"].items():
        assert abs(v - b["weight_norms"][k]) <= 1e-3 * max(1.0, abs(v)), k


@needs2
def test_fused_gemm_collectives(tmp_path):
    n = 2
    res = _run(n, ["fused"], str(tmp_path / "f.json"), ENV)
    assert res["native"] and res["world"] == n
    assert res["all_ranks_ok"], res


@needs2
def test_tensor_parallel_and_sharded_linear(tmp_path):
    res = _run(2, ["tp"], str(tmp_path / "t.json"), ENV)
    assert res["world"] == 2 and res["all_ranks_ok"], res


@needs2
def test_model_parallel_fc_on_fused_kernels(tmp_path):
    """``data_layout='model_parallel'`` fully-connected layers on a 2 x 1 process grid: the
    forward product stores its column block into both ranks' outputs from the GEMM epilogue
    (GEMM -> all-gather in one kernel), backward sums the input gradients with the
    all-reduce kernel.  Same losses and weights as one GPU."""
    single = _run(1, ["mpfc", "1", "4"], str(tmp_path / "a.json"), ENV)
    two = _run(2, ["mpfc", "2", "4"], str(tmp_path / "b.json"), ENV)
    assert two["world"] == 2
    for a, b in zip(single["losses"], two["losses"]):
        assert abs(a - b) <= 2e-2 * max(1.0, abs(a)), (single["losses"], two["losses"])
    for k, v in single["weight_norms"].items():
        assert abs(v - two["weight_norms"][k]) <= 1e-2 * max(1.0, abs(v)), k


@needs2
def test_partitioned_embedding_two_gpus(tmp_path):
    """The embedding table is split over two GPUs; rows are gathered from and gradients are
    added to their owners through peer memory.  Same losses and same trained table as the
    single-process run."""
    single = _run(1, ["distembed", "5"], str(tmp_path / "a.json"), {"LBANN_TEST_DEVICE": "cpu"})
    two = _run(2, ["distembed", "5"], str(tmp_path / "b.json"), ENV)
    assert two["world"] == 2 and two["status"] == 0
    for a, b in zip(single["losses"], two["losses"]):
        assert abs(a - b) <= 1e-3 * max(1.0, abs(a)), (single["losses"], two["losses"])
    assert max(abs(a - b) for a, b in zip(single["table"], two["table"])) < 1e-3


@needs2
@pytest.mark.parametrize("strategy", ["sendrecv_weights", "checkpoint_binary"])
def test_ltfb_two_trainers_on_gpus(tmp_path, strategy):
    """Two single-GPU trainers run tournaments; the one that cannot learn ends up with the
    learner's weights (weights travel GPU to GPU through the inter-trainer group)."""
    res = _run(2, ["ltfb", strategy], str(tmp_path / "l.json"), ENV)
    assert res["num_trainers"] == 2
    a, b = res["weights"]
    for k in a:
        assert abs(a[k] - b[k]) <= 1e-4 * max(1.0, abs(a[k])), (strategy, k, a, b)


@needs2
def test_checkpoint_restart_with_optimizer_state_for_owned_blocks(tmp_path):
    """Two GPUs, sharded update with momentum kept for the owned blocks only: a run that stops
    after two epochs and a second process that resumes from its checkpoint for the third end
    with the weights of an uninterrupted three-epoch run (the checkpoint gathers the state over
    the ranks, the restart takes every rank's share of it back)."""
    ref = _run(2, ["abort_restart", str(tmp_path / "ref"), "-1", "3"], str(tmp_path / "ref.json"), ENV, timeout=600)
    ck = str(tmp_path / "ck")
    first = _run(2, ["abort_restart", ck, "-1", "2"], str(tmp_path / "first.json"), ENV, timeout=600)
    again = _run(2, ["abort_restart", ck, "-1", "3"], str(tmp_path / "again.json"), ENV, timeout=600)
    assert first["epoch"] == 2 and again["epoch"] == 3 and again["step"] == ref["step"]
    assert ref["state_compact"] and ref["state_bytes"] <= 0.6 * ref["master_bytes"] + 2 * 65536
    for k, v in ref["weights"].items():
        assert abs(v - again["weights"][k]) <= 1e-4 * max(1.0, abs(v)), (k, v, again["weights"][k])
        assert abs(v - first["weights"][k]) > 0 or v == 0.0


needs4 = pytest.mark.skipif(torch.cuda.device_count() < 4, reason="needs four GPUs")


def _same_run(single, dist, loss_tol=1e-2, w_tol=5e-3):
    for a, b in zip(single["losses"], dist["losses"]):
        assert abs(a - b) <= loss_tol * max(1.0, abs(a)), (single["losses"], dist["losses"])
    for k, v in single["weight_norms"].items():
        assert abs(v - dist["weight_norms"][k]) <= w_tol * max(1.0, abs(v)), k


@needs4
@pytest.mark.parametrize("width,channels,graph", [("64", "16,32,32", ""),
                                                  ("128", "16,32,32,64,64", "graph")])
def test_distconv_four_gpus_matches_one(tmp_path, width, channels, graph):
    """Depth split over four GPUs: the two middle ranks exchange halo planes with a
    neighbour on either side.  Same losses and weights as one GPU."""
    steps = "8" if graph else "5"
    tail = [width, channels] + ([graph] if graph else [])
    single = _run(1, ["cosmoflow", "1", steps, "fp16"] + tail, str(tmp_path / "a.json"), STABLE)
    dist = _run(4, ["cosmoflow", "4", steps, "fp16"] + tail, str(tmp_path / "b.json"), STABLE)
    assert dist["status"] == 0 and dist["world"] == 4
    assert dist["interior_copies"] == 0, dist
    _same_run(single, dist)


@needs4
def test_sample_x_depth_partition_on_four_gpus(tmp_path):
    """Two sample groups of two depth ranks each, every group with its own symmetric
    memory for the halo exchange; the weight gradients are summed over all four."""
    tail = ["64", "16,32,32"]
    single = _run(1, ["cosmoflow", "1", "5", "fp16"] + tail, str(tmp_path / "a.json"), STABLE)
    dist = _run(4, ["cosmoflow", "2", "5", "fp16"] + tail, str(tmp_path / "b.json"), STABLE)
    assert dist["status"] == 0 and dist["world"] == 4
    _same_run(single, dist)


@needs4
def test_subgraph_parallel_branches_on_four_gpus(tmp_path):
    """Two sub-grids of two GPUs; tensors change grids through the row-scatter kernel."""
    single = _run(1, ["subgraph", "1", "4"], str(tmp_path / "a.json"), ENV)
    four = _run(4, ["subgraph", "2", "4"], str(tmp_path / "b.json"), ENV)
    assert four["world"] == 4
    _same_run(single, four, 2e-2, 1e-2)
