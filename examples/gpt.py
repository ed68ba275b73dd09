"""GPT decoder on synthetic tokens with the transformer parallelism switches
(applications/nlp/transformer of the reference: --fsdp, --fsdp-mlp, --ffn-parallel,
--lm-head-parallel, --layer-parallel).

    python examples/gpt.py --procs-per-node 8 --layers 24 --d-model 2048 --fsdp
"""
import argparse

import lbann
import lbann.contrib.args
import lbann.contrib.launcher
from lbann.models import parallelism
from lbann.models.transformer import construct_gpt_model


if __name__ == "__main__":
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    lbann.contrib.args.add_scheduler_arguments(ap, "gpt")
    lbann.contrib.args.add_training_arguments(ap, default_minibatch_size=64, default_epochs=1)
    parallelism.add_transformer_parallelism_arguments(ap)
    ap.add_argument("--layers", type=int, default=24)
    ap.add_argument("--d-model", type=int, default=2048)
    ap.add_argument("--heads", type=int, default=16)
    ap.add_argument("--seq", type=int, default=2048)
    ap.add_argument("--vocab", type=int, default=50304)
    ap.add_argument("--num-samples", type=int, default=1024)
    a = ap.parse_args()
    kw = lbann.contrib.args.get_scheduler_kwargs(a)
    world = (kw.get("nodes") or 1) * (kw.get("procs_per_node") or 1)
    model = construct_gpt_model(vocab_size=a.vocab, seq_len=a.seq, d_model=a.d_model, num_heads=a.heads,
                                num_layers=a.layers, ffn_dim=4 * a.d_model, num_epochs=a.num_epochs)
    extra = parallelism.apply_all(model, a, world)
    model.callbacks.extend([lbann.CallbackPrint(), lbann.CallbackTimer()])
    reader = lbann.reader_pb2.DataReader()
    r = reader.reader.add()
    r.name, r.role, r.shuffle, r.fraction_of_data_to_use = "synthetic", "train", False, 1.0
    r.synth_dimensions, r.num_samples, r.synth_distribution = str(a.seq + 1), a.num_samples, f"randint:{a.vocab}"
    trainer = lbann.Trainer(mini_batch_size=a.mini_batch_size)
    raise SystemExit(lbann.contrib.launcher.run(
        trainer, model, reader, lbann.Adam(learn_rate=3e-4, beta1=0.9, beta2=0.95, eps=1e-8),
        lbann_args=["--default_dtype=bf16", "--use_cuda_graph"] + list(extra), **kw))
