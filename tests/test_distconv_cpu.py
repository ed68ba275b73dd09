"""Depth-partitioned CosmoFlow on two gloo ranks reproduces the single-process run."""
import json
import os
import subprocess
import sys

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
WORKER = os.path.join(HERE, "_dist_worker.py")


def _run(nproc, args, out, env_extra=None, timeout=300):
    env = dict(os.environ)
    env.update(env_extra or {})
    env.setdefault("LBANN_TEST_DEVICE", "cpu")
    if nproc == 1:
        cmd = [sys.executable, WORKER] + args[:1] + [out] + args[1:]
    else:
        port = 29600 + os.getpid() % 300
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
               "--master-addr", "127.0.0.1", "--master-port", str(port), WORKER] + args[:1] + [out] + args[1:]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=timeout)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
    with open(out) as f:
        return json.load(f)


def test_distconv_two_ranks_matches_single(tmp_path):
    single = _run(1, ["cosmoflow", "1", "3"], str(tmp_path / "a.json"))
    dist = _run(2, ["cosmoflow", "2", "3"], str(tmp_path / "b.json"))
    assert dist["world"] == 2
    for a, b in zip(single["losses"], dist["losses"]):
        assert abs(a - b) <= 2e-4 * max(1.0, abs(a)), (single["losses"], dist["losses"])
    for k, v in single["weight_norms"].items():
        assert abs(v - dist["weight_norms"][k]) <= 1e-3 * max(1.0, abs(v)), k


def test_distconv_falls_back_to_sample_parallel_when_depth_runs_out(tmp_path):
    """Four ranks on a 16^3 volume with three conv/pool blocks: the last pooling would see
    one plane per rank, so it (and what follows) is computed sample-parallel after a
    redistribution; the result still matches the single-process run."""
    single = _run(1, ["cosmoflow", "1", "2", "float", "16"], str(tmp_path / "a.json"))
    dist = _run(4, ["cosmoflow", "4", "2", "float", "16"], str(tmp_path / "b.json"), timeout=600)
    assert dist["world"] == 4
    for a, b in zip(single["losses"], dist["losses"]):
        assert abs(a - b) <= 2e-4 * max(1.0, abs(a)), (single["losses"], dist["losses"])
    for k, v in single["weight_norms"].items():
        assert abs(v - dist["weight_norms"][k]) <= 1e-3 * max(1.0, abs(v)), k


def test_fused_gemm_collectives_gloo(tmp_path):
    """all-gather -> GEMM and GEMM -> reduce-scatter entry points on two CPU ranks (the
    torch.distributed fall-back path; the kernels themselves are covered on GPUs)."""
    res = _run(2, ["fused"], str(tmp_path / "f.json"))
    assert res["world"] == 2 and res["all_ranks_ok"], res


def test_tensor_parallel_and_sharded_linear_gloo(tmp_path):
    """Column-/row-parallel FFN pair and FSDP-style sharded linear layer on two CPU ranks
    reproduce the dense fp32 forward values and all gradients."""
    res = _run(2, ["tp"], str(tmp_path / "t.json"))
    assert res["world"] == 2 and res["all_ranks_ok"], res


def test_model_parallel_fully_connected_matches_single(tmp_path):
    """FullyConnected layers with data_layout='model_parallel' on a 2 x 1 process grid give
    the losses and weights of the single-process run."""
    single = _run(1, ["mpfc", "1", "4"], str(tmp_path / "a.json"))
    grid = _run(2, ["mpfc", "2", "4"], str(tmp_path / "b.json"))
    assert grid["world"] == 2
    for a, b in zip(single["losses"], grid["losses"]):
        assert abs(a - b) <= 1e-4 * max(1.0, abs(a)), (single["losses"], grid["losses"])
    for k, v in single["weight_norms"].items():
        assert abs(v - grid["weight_norms"][k]) <= 1e-4 * max(1.0, abs(v)), k


@pytest.mark.parametrize("strategy", ["checkpoint_binary", "sendrecv_weights", "truncation"])
def test_ltfb_two_trainers(tmp_path, strategy):
    """Two single-rank trainers, one of which cannot learn (zero learning rate): after the
    tournaments both hold the learner's weights."""
    res = _run(2, ["ltfb", strategy], str(tmp_path / "l.json"))
    assert res["num_trainers"] == 2
    a, b = res["weights"]
    for k in a:
        assert abs(a[k] - b[k]) <= 1e-5 * max(1.0, abs(a[k])), (strategy, k, a, b)


def test_sharded_weights_fully_connected_matches_single(tmp_path):
    """A fully-connected layer whose weights carry the ``sharded`` flag, on two data-parallel
    ranks (all-gather -> GEMM forward, reduce-scattered weight gradient), follows the
    single-process trajectory."""
    single = _run(1, ["mpfc", "1", "4", "sharded"], str(tmp_path / "a.json"))
    two = _run(2, ["mpfc", "1", "4", "sharded"], str(tmp_path / "b.json"))
    assert two["world"] == 2
    for a, b in zip(single["losses"], two["losses"]):
        assert abs(a - b) <= 2e-4 * max(1.0, abs(a)), (single["losses"], two["losses"])
    for k, v in single["weight_norms"].items():
        assert abs(v - two["weight_norms"][k]) <= 2e-4 * max(1.0, abs(v)), k


def test_partitioned_embedding_with_sparse_sgd_matches_single_rank(tmp_path):
    """dist_embedding with its own sparse SGD: two ranks (replicated table, gathered
    gradients on CPU) train the same table as one rank; indices beyond the table give zeros."""
    single = _run(1, ["distembed", "5"], str(tmp_path / "a.json"))
    two = _run(2, ["distembed", "5"], str(tmp_path / "b.json"))
    assert two["world"] == 2
    for a, b in zip(single["losses"], two["losses"]):
        assert abs(a - b) <= 1e-4 * max(1.0, abs(a)), (single["losses"], two["losses"])
    assert max(abs(a - b) for a, b in zip(single["table"], two["table"])) < 1e-4
    assert single["losses"][-1] < single["losses"][0]


def test_subgraph_parallel_branches_on_two_grids(tmp_path):
    """Sub-graph parallelism on four CPU ranks split into two grids: the two branches run
    on ranks {0, 1} and {2, 3}, untagged layers inherit their parents' grid, the join runs
    on all ranks; tensors cross between the grids sample by sample.  Same training
    trajectory as one process."""
    single = _run(1, ["subgraph", "1", "4"], str(tmp_path / "a.json"))
    four = _run(4, ["subgraph", "2", "4"], str(tmp_path / "b.json"), timeout=600)
    assert four["world"] == 4
    assert four["tags"] == {"branch1_sin": 1, "branch1_fc": 1, "branch2_cos": 2, "branch2_fc": 2,
                            "join": 0, "head": 0}
    for a, b in zip(single["losses"], four["losses"]):
        assert abs(a - b) <= 2e-4 * max(1.0, abs(a)), (single["losses"], four["losses"])
    for k, v in single["weight_norms"].items():
        assert abs(v - four["weight_norms"][k]) <= 1e-4 * max(1.0, abs(v)), k


def test_kfac_inverses_spread_over_the_ranks(tmp_path):
    """distribute_precondition_compute: every factor is inverted by one rank only and the
    others receive it; the training trajectory is the one of the replicated computation."""
    rep = _run(2, ["kfac", "0", "4"], str(tmp_path / "a.json"))
    dist = _run(2, ["kfac", "1", "4"], str(tmp_path / "b.json"))
    # 3 blocks: fc1 and fc2 have two factors, bn1 one -> 5 inverses per step
    assert rep["inverses"] == [20.0, 20.0]
    assert sorted(dist["inverses"]) == [4.0, 16.0] and sum(dist["inverses"]) == 20.0
    for k, v in rep["weight_norms"].items():
        assert abs(v - dist["weight_norms"][k]) <= 1e-5 * max(1.0, abs(v)), k


def test_kfac_asynchronous_inverses_keep_the_ranks_identical(tmp_path):
    """Distributed and asynchronous: the owner inverts beside the next step, every rank installs
    the result at the same (following) step, so the replicas never drift apart."""
    res = _run(2, ["kfac", "1", "6", "1"], str(tmp_path / "a.json"))
    sync = _run(2, ["kfac", "1", "6", "0"], str(tmp_path / "b.json"))
    assert res["world"] == 2 and sum(res["inverses"]) == 30.0 and sorted(res["inverses"]) == [6.0, 24.0]
    assert res["installs"] == 5 * 4                # steps 1..4 started jobs that a later step installed
    a, b = res["all_weight_norms"]
    for k, v in a.items():
        if "running" not in k:                     # batch-norm statistics are local to a rank here
            assert abs(v - b[k]) <= 1e-9 * max(1.0, abs(v)), k
    # stale-by-one inverses give a slightly different, equally good trajectory
    assert res["objective"] < 1.5 * sync["objective"], (res["objective"], sync["objective"])


def test_subgraph_transformer_heads_on_two_grids(tmp_path):
    """Attention heads of an encoder dealt onto two sub-grids of two ranks each: same
    trajectory as one process running all heads."""
    single = _run(1, ["subgraph_transformer", "1", "3"], str(tmp_path / "a.json"))
    four = _run(4, ["subgraph_transformer", "2", "3"], str(tmp_path / "b.json"), timeout=900)
    assert four["world"] == 4 and four["tags"] == [0, 1, 2]
    assert sorted(set(four["head_tags"].values())) == [1, 2] and len(four["head_tags"]) == 4
    for a, b in zip(single["losses"], four["losses"]):
        assert abs(a - b) <= 2e-4 * max(1.0, abs(a)), (single["losses"], four["losses"])
    for k, v in single["weight_norms"].items():
        assert abs(v - four["weight_norms"][k]) <= 1e-4 * max(1.0, abs(v)), k


def test_sample_x_depth_partition_on_four_ranks(tmp_path):
    """depth_groups = 2 on four ranks: two sample groups of two depth ranks each (the
    left-over ranks multiply the sample groups).  Same results as one process."""
    single = _run(1, ["cosmoflow", "1", "3"], str(tmp_path / "a.json"))
    dist = _run(4, ["cosmoflow", "2", "3"], str(tmp_path / "b.json"), timeout=600)
    assert dist["world"] == 4
    for a, b in zip(single["losses"], dist["losses"]):
        assert abs(a - b) <= 2e-4 * max(1.0, abs(a)), (single["losses"], dist["losses"])
    for k, v in single["weight_norms"].items():
        assert abs(v - dist["weight_norms"][k]) <= 1e-3 * max(1.0, abs(v)), k


def test_distconv_eight_ranks_match_single(tmp_path):
    """Depth split over eight ranks, mini-batch 8: the layout of the 8-GPU CosmoFlow run in
    small (local depth 4 -> 2 -> 1, the last convolution sees ONE plane per rank with both
    neighbours' halos, then the tensor is gathered to one sample per rank)."""
    env = {"LBANN_TEST_MINI_BATCH": "8", "OMP_NUM_THREADS": "2"}
    single = _run(1, ["cosmoflow", "1", "2"], str(tmp_path / "a.json"), env)
    dist = _run(8, ["cosmoflow", "8", "2"], str(tmp_path / "b.json"), env, timeout=900)
    assert dist["world"] == 8
    for a, b in zip(single["losses"], dist["losses"]):
        assert abs(a - b) <= 2e-4 * max(1.0, abs(a)), (single["losses"], dist["losses"])
    for k, v in single["weight_norms"].items():
        assert abs(v - dist["weight_norms"][k]) <= 1e-3 * max(1.0, abs(v)), k


def test_distconv_depth_x_height_grid_matches_single(tmp_path):
    """Four ranks as a 2 x 2 grid over depth and height: halo planes are exchanged along
    depth, then halo rows (with the corners) along height; where the extents run out the
    bricks are gathered to sample-parallel.  Same losses and weights as one process."""
    single = _run(1, ["cosmoflow", "1", "3"], str(tmp_path / "a.json"))
    grid = _run(4, ["cosmoflow", "2", "3"], str(tmp_path / "b.json"), {"LBANN_TEST_HEIGHT_GROUPS": "2"},
                timeout=600)
    assert grid["world"] == 4 and grid["halo_bytes"] > 0
    for a, b in zip(single["losses"], grid["losses"]):
        assert abs(a - b) <= 2e-4 * max(1.0, abs(a)), (single["losses"], grid["losses"])
    for k, v in single["weight_norms"].items():
        assert abs(v - grid["weight_norms"][k]) <= 1e-3 * max(1.0, abs(v)), k


@pytest.mark.parametrize("ranks,depth,height,width", [(2, 1, 1, 2), (4, 1, 2, 2), (8, 2, 2, 2)])
def test_distconv_width_partitions_match_single(tmp_path, ranks, depth, height, width):
    """Width alone, a height x width grid and a 2 x 2 x 2 grid over all three dimensions (edge and
    corner regions arrive over two and three hops): same losses and weights as one process."""
    single = _run(1, ["cosmoflow", "1", "3"], str(tmp_path / "a.json"))
    grid = _run(ranks, ["cosmoflow", str(depth), "3"], str(tmp_path / "b.json"),
                {"LBANN_TEST_HEIGHT_GROUPS": str(height), "LBANN_TEST_WIDTH_GROUPS": str(width)}, timeout=900)
    assert grid["world"] == ranks and grid["halo_bytes"] > 0
    for a, b in zip(single["losses"], grid["losses"]):
        assert abs(a - b) <= 2e-4 * max(1.0, abs(a)), (single["losses"], grid["losses"])
    for k, v in single["weight_norms"].items():
        assert abs(v - grid["weight_norms"][k]) <= 1e-3 * max(1.0, abs(v)), k


@pytest.mark.parametrize("ranks,depth,height", [(2, 2, 1), (2, 1, 2), (4, 2, 2)])
def test_unet_on_spatial_partitions_matches_single(tmp_path, ranks, depth, height):
    """A small 3-D U-Net (convolution + batch norm over all ranks + ReLU, max pooling, 2x
    up-convolutions, skip concatenations, per-voxel labels sliced like the volume, softmax
    cross-entropy summed over the bricks) split along depth, along height, and on a grid."""
    single = _run(1, ["unet", "1", "1", "4"], str(tmp_path / "a.json"))
    dist = _run(ranks, ["unet", str(depth), str(height), "4"], str(tmp_path / "b.json"), timeout=900)
    assert dist["world"] == ranks
    for a, b in zip(single["losses"], dist["losses"]):
        assert abs(a - b) <= 1e-4 * max(1.0, abs(a)), (single["losses"], dist["losses"])
    assert dist["losses"][-1] < dist["losses"][0]
    for k, v in single["weight_norms"].items():
        assert abs(v - dist["weight_norms"][k]) <= 1e-4 * max(1.0, abs(v)), k


@pytest.mark.parametrize("mini_batch", ["6", "2"])
def test_distconv_uneven_and_empty_sample_shares(tmp_path, mini_batch):
    """Four ranks whose sample-parallel tail gets unequal shares of a mini-batch (6 samples:
    2, 2, 1, 1) or none at all on some ranks (2 samples): shares are padded to a common
    size for the way back to the spatial layout, and layers run on empty shares."""
    env = {"LBANN_TEST_MINI_BATCH": mini_batch, "LBANN_TEST_LR": "0.001"}
    single = _run(1, ["cosmoflow", "1", "3", "float", "16"], str(tmp_path / "a.json"), env)
    dist = _run(4, ["cosmoflow", "4", "3", "float", "16"], str(tmp_path / "b.json"), env, timeout=600)
    assert dist["world"] == 4
    for a, b in zip(single["losses"], dist["losses"]):
        assert abs(a - b) <= 2e-4 * max(1.0, abs(a)), (single["losses"], dist["losses"])
    for k, v in single["weight_norms"].items():
        assert abs(v - dist["weight_norms"][k]) <= 1e-3 * max(1.0, abs(v)), k


def test_layer_parallel_placement_on_two_subgrids(tmp_path):
    """GPT blocks 0-1 on sub-grid 1 and blocks 2-3 on sub-grid 2 (four ranks, two per grid;
    activations move between the rank subsets at the block boundary): same losses and
    weights as one process."""
    single = _run(1, ["layer_parallel", "1", "3"], str(tmp_path / "a.json"))
    four = _run(4, ["layer_parallel", "2", "3"], str(tmp_path / "b.json"), timeout=600)
    assert four["world"] == 4 and four["tags"] == [0, 1, 2] and four["grids"] == 2
    for a, b in zip(single["losses"], four["losses"]):
        assert abs(a - b) <= 2e-4 * max(1.0, abs(a)), (single["losses"], four["losses"])
    for k, v in single["weight_norms"].items():
        assert abs(v - four["weight_norms"][k]) <= 1e-4 * max(1.0, abs(v)), k


@pytest.mark.parametrize("ranks", [2, 4])
def test_token_parallel_attention_block_matches_single(tmp_path, ranks):
    """channel_groups = 2 on the layers of an attention + MLP block over [tokens, features]
    tensors: tokens are split over two ranks, channel-wise products / activations / softmax stay
    local, the score and context products gather keys and values, the head runs
    sample-parallel.  With four ranks there are two sample groups (and uneven shares)."""
    single = _run(1, ["token_parallel", "1", "4"], str(tmp_path / "a.json"))
    dist = _run(ranks, ["token_parallel", "2", "4"], str(tmp_path / "b.json"), timeout=600)
    assert dist["world"] == ranks and dist["sample_groups"] == ranks // 2
    assert {"q", "k", "v", "scores", "probs", "context", "up", "down"} <= set(dist["partitioned"])
    assert dist["losses"][-1] < dist["losses"][0]
    for a, b in zip(single["losses"], dist["losses"]):
        assert abs(a - b) <= 2e-4 * max(1.0, abs(a)), (single["losses"], dist["losses"])
    for k, v in single["weight_norms"].items():
        assert abs(v - dist["weight_norms"][k]) <= 1e-4 * max(1.0, abs(v)), k


@pytest.mark.parametrize("ranks,groups", [(2, 2), (4, 4), (4, 2)])
def test_channel_filter_parallel_convolutions_match_single(tmp_path, ranks, groups):
    """channel_groups == filter_groups on convolutions, activations and poolings: every rank
    gathers the input channels, applies its block of filters and keeps its block of output
    channels; the batch norm between them runs sample-parallel.  Same losses and weights as one
    process (4 ranks with 2 groups: two sample groups)."""
    single = _run(1, ["filter_parallel", "1", "4"], str(tmp_path / "a.json"))
    dist = _run(ranks, ["filter_parallel", str(groups), "4"], str(tmp_path / "b.json"), timeout=600)
    assert dist["world"] == ranks and dist["sample_groups"] == ranks // groups
    assert {"conv1", "act1", "pool1", "conv2", "act2", "pool2"} <= set(dist["partitioned"])
    assert "bn" not in dist["partitioned"]
    for a, b in zip(single["losses"], dist["losses"]):
        assert abs(a - b) <= 2e-4 * max(1.0, abs(a)), (single["losses"], dist["losses"])
    for k, v in single["weight_norms"].items():
        assert abs(v - dist["weight_norms"][k]) <= 1e-4 * max(1.0, abs(v)), k
