"""Application models of the reference's ``applications/`` tree, built through the front end:
auto-encoders and a variational auto-encoder (autoencoders/, ATOM), a hinge GAN trained by
alternating updates (gan/mnist), DenseNet (vision/densenet.py), a character GRU language
model (ATOM/train_atom_char_rnn.py), a dense-graph GCN classifier (graph/GNN), a siamese patch
network with shared towers (selfsupervised/), the CANDLE Pilot-1 combo regressor
(CANDLE/pilot1/combo.py), the JAG Wasserstein auto-encoder (physics/ICF/jag_models.py), node2vec
skip-gram with negative sampling (graph/node2vec), a 3-D voxel auto-encoder (MOF/) and an
image regressor (physics/HRRL).
Every builder returns an ``lbann.Model`` reading the data fields named in its docstring.
"""
from __future__ import annotations

from typing import Sequence

from ..frontend import core as L
from ..modules import ConvolutionModule, Convolution2dModule, FullyConnectedModule, Module
from ..modules.graph import DenseGCNConv
from ..modules.rnn import GRU


def _mlp(x, sizes: Sequence[int], name: str, activation=L.Relu, last_activation=None, dropout=None):
    for i, n in enumerate(sizes):
        act = activation if i < len(sizes) - 1 else last_activation
        x = FullyConnectedModule(n, activation=act, name=f"{name}_fc{i}")(x)
        if dropout and i < len(sizes) - 1:
            x = L.Dropout(x, keep_prob=1.0 - dropout, name=f"{name}_drop{i}")
    return x


# ----------------------------------------------------------------------------- auto-encoders
def construct_autoencoder(input_dims=(1, 28, 28), kind="dense", hidden=(1000, 500, 250, 30), num_epochs=1):
    """``samples`` -> reconstruction.  ``dense``: mirrored fully-connected stacks with a sigmoid
    output; ``conv``: two stride-2 convolutions down, two transposed convolutions up.  Loss
    and metric: mean squared error against the input (applications/autoencoders/mnist)."""
    x = L.Input(data_field="samples", name="image")
    n = 1
    for d in input_dims:
        n *= d
    if kind == "dense":
        h = L.Reshape(x, dims=[n], name="flat")
        h = _mlp(h, hidden, "encode", last_activation=None)
        h = _mlp(h, tuple(reversed(hidden[:-1])) + (n,), "decode", last_activation=L.Sigmoid)
        recon, target = h, L.Reshape(x, dims=[n], name="target")
    else:
        c = input_dims[0]
        h = Convolution2dModule(16, 3, stride=2, padding=1, activation=L.Relu, name="enc1")(x)
        h = Convolution2dModule(32, 3, stride=2, padding=1, activation=L.Relu, name="enc2")(h)
        h = ConvolutionModule(2, 16, 2, stride=2, transpose=True, activation=L.Relu, name="dec1")(h)
        h = ConvolutionModule(2, c, 2, stride=2, transpose=True, activation=L.Sigmoid, name="dec2")(h)
        recon, target = h, x
    mse = L.MeanSquaredError(recon, target, name="reconstruction_error")
    return L.Model(num_epochs, layers=list(L.traverse_layer_graph(x)),
                   objective_function=L.ObjectiveFunction([mse]),
                   metrics=[L.Metric(mse, name="reconstruction error")])


def construct_vae(input_size=784, hidden=(512, 256), latent=20, kl_weight=1.0, num_epochs=1):
    """Variational auto-encoder on flat ``samples`` in [0, 1]: encoder -> (mean, log variance),
    z = mean + exp(log variance / 2) * N(0, 1), decoder logits; objective = sigmoid binary
    cross-entropy of the reconstruction + ``kl_weight`` * KL(q(z|x) || N(0, 1))
    (the structure of applications/ATOM/models/vae.py with dense encoders)."""
    x = L.Reshape(L.Input(data_field="samples", name="image"), dims=[input_size], name="x")
    h = _mlp(x, hidden, "vae_enc", last_activation=L.Relu)
    mu = FullyConnectedModule(latent, name="vae_mu")(h)
    logvar = FullyConnectedModule(latent, name="vae_logvar")(h)
    eps = L.Gaussian(mean=0.0, stdev=1.0, neuron_dims=[latent], name="vae_eps")
    std = L.Exp(L.Scale(logvar, constant=0.5, name="vae_half_logvar"), name="vae_std")
    z = L.Add(mu, L.Multiply(std, eps, name="vae_noise"), name="vae_z")
    logits = _mlp(z, tuple(reversed(hidden)) + (input_size,), "vae_dec", last_activation=None)
    bce = L.Reduction(L.SigmoidBinaryCrossEntropy(logits, x, name="vae_bce_elem"), mode="sum", name="vae_bce")
    # KL = -1/2 sum(1 + logvar - mu^2 - exp(logvar))
    kl_terms = L.WeightedSum([logvar, L.Square(mu, name="vae_mu2"), L.Exp(logvar, name="vae_var")],
                             scaling_factors=[-0.5, 0.5, 0.5], name="vae_kl_terms")
    kl = L.AddConstant(L.Reduction(kl_terms, mode="sum", name="vae_kl_sum"), constant=-0.5 * latent, name="vae_kl")
    return L.Model(num_epochs, layers=list(L.traverse_layer_graph(x)),
                   objective_function=L.ObjectiveFunction([L.LayerTerm(bce), L.LayerTerm(kl, scale=kl_weight)]),
                   metrics=[L.Metric(bce, name="reconstruction"), L.Metric(kl, name="kl divergence")])


# ----------------------------------------------------------------------------------- GAN
class _Generator(Module):
    def __init__(self, out_size, hidden, name="gen"):
        super().__init__()
        self.stack = [FullyConnectedModule(n, activation=L.Relu, name=f"{name}_fc{i}")
                      for i, n in enumerate(hidden)]
        self.out = FullyConnectedModule(out_size, activation=L.Sigmoid, name=f"{name}_out")

    def forward(self, z):
        for m in self.stack:
            z = m(z)
        return self.out(z)


class _Discriminator(Module):
    def __init__(self, hidden, name="disc"):
        super().__init__()
        self.stack = [FullyConnectedModule(n, name=f"{name}_fc{i}") for i, n in enumerate(hidden)]
        self.out = FullyConnectedModule(1, name=f"{name}_out")

    def forward(self, x):
        for m in self.stack:                  # shared weights: applied to real and generated samples
            x = L.LeakyRelu(m(x), negative_slope=0.2)
        return self.out(x)


def construct_gan(sample_size=784, noise_size=16, hidden=(256, 256), num_epochs=1, disc_iters=1, gen_iters=1):
    """Hinge GAN on flat ``samples``: loss = relu(1 - D(real)) + relu(1 + D(fake)) for the
    discriminator and -D(fake) for the generator, each behind an ``IdentityZero`` layer (which
    passes nothing while its side is frozen); the ``alternate_updates`` callback freezes the
    discriminator's and the generator's layers in turn (applications/gan/mnist/gan_model.py)."""
    gen, disc = _Generator(sample_size, hidden), _Discriminator(tuple(reversed(hidden)))
    real = L.Reshape(L.Input(data_field="samples", name="real_samples"), dims=[sample_size], name="real")
    fake = gen(L.Gaussian(mean=0.0, stdev=1.0, neuron_dims=[noise_size], name="gen_noise"))
    real_out, fake_out = disc(real), disc(fake)
    real_loss = L.Relu(L.AddConstant(L.Negative(real_out), constant=1.0), name="disc_real_hinge")
    fake_loss = L.Relu(L.AddConstant(fake_out, constant=1.0), name="disc_fake_hinge")
    disc_loss = L.IdentityZero(L.Add(real_loss, fake_loss), name="disc_loss")
    gen_loss = L.IdentityZero(L.Negative(fake_out), name="gen_loss")
    loss = L.Add(disc_loss, gen_loss, name="gan_loss")
    layers = list(L.traverse_layer_graph(loss))
    disc_layers = [disc_loss.name] + [l.name for l in layers if l.weights and l.name.startswith("disc_")]
    gen_layers = [gen_loss.name] + [l.name for l in layers if l.weights and l.name.startswith("gen_")]
    cb = L.CallbackAlternateUpdates(layers_1=" ".join(disc_layers), layers_2=" ".join(gen_layers),
                                    iters_1=disc_iters, iters_2=gen_iters)
    return L.Model(num_epochs, layers=layers, objective_function=L.ObjectiveFunction([loss]),
                   metrics=[L.Metric(disc_loss, name="discriminator loss"), L.Metric(gen_loss, name="generator loss")],
                   callbacks=[cb])


# ------------------------------------------------------------------------------ DenseNet
def construct_densenet(num_classes=1000, growth=32, blocks=(6, 12, 24, 16), init_features=64,
                       bn_statistics_group_size=1, small_input=False, num_epochs=1):
    """DenseNet-121 by default (blocks 6-12-24-16, growth 32): every layer of a dense block is
    BN-ReLU-1x1(4k)-BN-ReLU-3x3(k) on the concatenation of all earlier outputs; transitions
    halve channels and resolution (applications/vision/densenet.py).  ``small_input`` replaces
    the 7x7 / stride-2 stem and its pooling by one 3x3 convolution (CIFAR-size images)."""
    g = bn_statistics_group_size

    def bn_relu(x, name):
        return L.Relu(L.BatchNormalization(x, statistics_group_size=g, decay=0.9, epsilon=1e-5, name=name + "_bn"),
                      name=name + "_relu")

    img = L.Input(data_field="samples", name="image")
    lab = L.Input(data_field="labels", name="label")
    if small_input:
        x = Convolution2dModule(init_features, 3, padding=1, bias=False, name="stem_conv")(img)
    else:
        x = Convolution2dModule(init_features, 7, stride=2, padding=3, bias=False, name="stem_conv")(img)
        x = bn_relu(x, "stem")
        x = L.Pooling(x, num_dims=2, has_vectors=False, pool_dims_i=3, pool_pads_i=1, pool_strides_i=2,
                      pool_mode="max", name="stem_pool")
    ch = init_features
    for b, n in enumerate(blocks):
        for i in range(n):
            name = f"block{b}_layer{i}"
            y = Convolution2dModule(4 * growth, 1, bias=False, name=name + "_conv1")(bn_relu(x, name + "_a"))
            y = Convolution2dModule(growth, 3, padding=1, bias=False, name=name + "_conv2")(bn_relu(y, name + "_b"))
            x = L.Concatenation([x, y], axis=0, name=name + "_cat")
            ch += growth
        if b < len(blocks) - 1:
            ch //= 2
            x = Convolution2dModule(ch, 1, bias=False, name=f"trans{b}_conv")(bn_relu(x, f"trans{b}"))
            x = L.Pooling(x, num_dims=2, has_vectors=False, pool_dims_i=2, pool_pads_i=0, pool_strides_i=2,
                          pool_mode="average", name=f"trans{b}_pool")
    x = L.ChannelwiseMean(bn_relu(x, "final"), name="global_pool")
    probs = L.Softmax(FullyConnectedModule(num_classes, name="classifier")(x), name="probs")
    ce = L.CrossEntropy(probs, lab, name="cross_entropy")
    acc = L.CategoricalAccuracy(probs, lab, name="top1")
    return L.Model(num_epochs, layers=list(L.traverse_layer_graph([img, lab])),
                   objective_function=L.ObjectiveFunction([ce, L.L2WeightRegularization(scale=1e-4)]),
                   metrics=[L.Metric(acc, name="accuracy", unit="%")])


# ------------------------------------------------------------------------- character GRU
def construct_char_rnn(vocab_size, sequence_length, embedding_size=64, hidden_size=128, num_layers=1,
                       pad_index=-1, num_epochs=1):
    """Next-character model over integer ``samples`` of ``sequence_length`` tokens: embedding ->
    GRU -> per-position softmax over the vocabulary; objective = mean cross-entropy of tokens
    1..n given 0..n-1 (applications/ATOM/train_atom_char_rnn.py)."""
    n = sequence_length
    tokens = L.Identity(L.Input(data_field="samples", name="tokens"), name="token_ids")
    emb = L.Embedding(tokens, num_embeddings=vocab_size, embedding_dim=embedding_size,
                      padding_idx=pad_index, name="char_embedding")
    head = L.Slice(emb, axis=0, slice_points=[0, n - 1], name="inputs")                    # tokens 0..n-2
    h0 = L.Constant(value=0.0, num_neurons=[num_layers, hidden_size], name="h0")
    out = GRU(hidden_size, num_layers=num_layers, name="char_gru")(head, h0)              # [n-1, hidden]
    logits = L.ChannelwiseFullyConnected(out, output_channel_dims=[vocab_size], name="char_logits")
    # [positions, vocabulary] -> channels = vocabulary: per-position softmax, integer targets
    probs = L.Softmax(L.TensorPermute(logits, axes=[1, 0], name="char_logits_t"), softmax_mode="channel",
                      name="char_probs")
    target = L.Identity(L.Slice(tokens, axis=0, slice_points=[1, n], name="targets"), name="next_chars")
    ce = L.Scale(L.CrossEntropy(probs, target, use_labels=True, name="char_ce_sum"), constant=1.0 / (n - 1),
                 name="char_ce")
    return L.Model(num_epochs, layers=list(L.traverse_layer_graph(tokens)),
                   objective_function=L.ObjectiveFunction([ce]),
                   metrics=[L.Metric(ce, name="cross entropy per character")])


# --------------------------------------------------------------------- dense-graph classifier
def construct_dense_gcn(num_nodes, num_features, num_classes, hidden=(32, 32), num_epochs=1):
    """Graph classification on dense graphs: ``samples`` = [node features (nodes x features),
    adjacency (nodes x nodes)] flattened and concatenated, ``labels`` one-hot.  GCN layers,
    mean over the nodes, a linear classifier (applications/graph/GNN/Dense_Graph_Trainer.py)."""
    s = L.Input(data_field="samples", name="graph")
    lab = L.Input(data_field="labels", name="graph_label")
    pieces = L.Slice(s, axis=0, slice_points=[0, num_nodes * num_features, num_nodes * (num_features + num_nodes)],
                     name="graph_slice")
    x = L.Reshape(L.Identity(pieces), dims=[num_nodes, num_features], name="node_features")
    adj = L.Reshape(L.Identity(pieces), dims=[num_nodes, num_nodes], name="adjacency")
    fin = num_features
    for i, h in enumerate(hidden):
        x = L.Relu(DenseGCNConv(fin, h, name=f"gcn{i}")(x, adj), name=f"gcn{i}_relu")
        fin = h
    pooled = L.Reshape(L.MatMul(L.Constant(value=1.0 / num_nodes, num_neurons=[1, num_nodes], name="mean_row"), x,
                                name="node_mean"), dims=[fin])
    probs = L.Softmax(FullyConnectedModule(num_classes, name="graph_classifier")(pooled), name="graph_probs")
    ce = L.CrossEntropy(probs, lab, name="graph_ce")
    acc = L.CategoricalAccuracy(probs, lab, name="graph_acc")
    return L.Model(num_epochs, layers=list(L.traverse_layer_graph([s, lab])),
                   objective_function=L.ObjectiveFunction([ce]), metrics=[L.Metric(acc, name="accuracy", unit="%")])


# ----------------------------------------------------------------------------- siamese patches
def construct_siamese(num_patches=3, patch_dims=(3, 32, 32), num_classes=6, embed=64, num_epochs=1):
    """Self-supervised patch-order prediction: ``samples`` holds ``num_patches`` patches stacked
    along channels; one convolutional tower (shared weights) embeds every patch, the
    concatenated embeddings classify which permutation produced the order
    (applications/selfsupervised/pretrain_siamese.py)."""
    c = patch_dims[0]
    img = L.Input(data_field="samples", name="patches")
    lab = L.Input(data_field="labels", name="permutation")
    pieces = L.Slice(img, axis=0, slice_points=[i * c for i in range(num_patches + 1)], name="patch_slice")
    tower = [Convolution2dModule(16, 3, stride=2, padding=1, activation=L.Relu, name="tower_conv1"),
             Convolution2dModule(32, 3, stride=2, padding=1, activation=L.Relu, name="tower_conv2"),
             FullyConnectedModule(embed, activation=L.Relu, name="tower_fc")]
    feats = []
    for _ in range(num_patches):
        h = L.Identity(pieces)
        for m in tower:
            h = m(h)
        feats.append(h)
    joint = L.Concatenation(feats, axis=0, name="joint_embedding")
    probs = L.Softmax(_mlp(joint, (128, num_classes), "head"), name="perm_probs")
    ce = L.CrossEntropy(probs, lab, name="perm_ce")
    acc = L.CategoricalAccuracy(probs, lab, name="perm_acc")
    return L.Model(num_epochs, layers=list(L.traverse_layer_graph([img, lab])),
                   objective_function=L.ObjectiveFunction([ce]), metrics=[L.Metric(acc, name="accuracy", unit="%")])


# ------------------------------------------------------------------------------ CANDLE combo
def construct_candle_combo(cell_features=942, drug_features=3820, hidden=(1000, 1000, 1000), dropout=0.0,
                           num_epochs=1):
    """Pilot-1 drug-pair response regressor: ``samples`` = [cell line expression | drug 1
    descriptors | drug 2 descriptors]; one feature tower per input kind, the two drugs share
    theirs; the concatenated features go through a residual dense stack to one growth value
    (``responses``), mean squared error (applications/CANDLE/pilot1/combo.py)."""
    s = L.Input(data_field="samples", name="combo_input")
    y = L.Input(data_field="responses", name="growth")
    pts = [0, cell_features, cell_features + drug_features, cell_features + 2 * drug_features]
    pieces = L.Slice(s, axis=0, slice_points=pts, name="combo_slice")
    cell = _mlp(L.Identity(pieces), hidden, "cell_tower", last_activation=L.Relu, dropout=dropout)
    drug_tower = [FullyConnectedModule(n, activation=L.Relu, name=f"drug_tower_fc{i}") for i, n in enumerate(hidden)]
    drugs = []
    for _ in range(2):
        h = L.Identity(pieces)
        for m in drug_tower:
            h = m(h)
        drugs.append(h)
    h = L.Concatenation([cell] + drugs, axis=0, name="combo_features")
    for i, n in enumerate(hidden):
        z = FullyConnectedModule(n, activation=L.Relu, name=f"combo_fc{i}")(h)
        h = L.Add(h, z, name=f"combo_res{i}") if i > 0 else z             # residual from the second layer on
    pred = FullyConnectedModule(1, name="combo_out")(h)
    mse = L.MeanSquaredError(pred, y, name="combo_mse")
    mae = L.MeanAbsoluteError(pred, y, name="combo_mae")
    return L.Model(num_epochs, layers=list(L.traverse_layer_graph([s, y])),
                   objective_function=L.ObjectiveFunction([mse]),
                   metrics=[L.Metric(mse, name="mse"), L.Metric(mae, name="mae")])


# ----------------------------------------------------------------------------------- JAG WAE
def construct_jag_wae(sample_size=16399, latent=20, enc_hidden=(32, 256, 128), disc_hidden=(128, 16),
                      adversarial_weight=0.01, num_epochs=1):
    """Wasserstein auto-encoder of JAG outputs (scalars + image pixels as flat ``samples``):
    encoder -> latent -> decoder with a reconstruction MSE, plus a latent discriminator that
    tells encoded samples from N(0, 1) draws; the encoder is also trained to fool a copy of it
    that has no optimizer and is refreshed by the ``replace_weights`` callback
    (applications/physics/ICF/jag_models.py)."""
    x = L.Input(data_field="samples", name="jag_sample")
    z = _mlp(x, tuple(enc_hidden) + (latent,), "wae_enc", activation=L.Tanh)
    recon = _mlp(z, tuple(reversed(enc_hidden)) + (sample_size,), "wae_dec", activation=L.Tanh)
    mse = L.MeanSquaredError(recon, x, name="wae_recon")
    prior = L.Gaussian(mean=0.0, stdev=1.0, neuron_dims=[latent], name="wae_prior")
    sizes = tuple(disc_hidden) + (1,)

    def weights(tag, optimizer=None):
        kw = {} if optimizer is None else {"optimizer": optimizer}
        return [[L.Weights(initializer=L.HeNormalInitializer(), name=f"wae_{tag}_fc{i}_matrix", **kw),
                 L.Weights(initializer=L.ConstantInitializer(value=0.0), name=f"wae_{tag}_fc{i}_bias", **kw)]
                for i in range(len(sizes))]

    def disc(v, ws, tag):
        for i, n in enumerate(sizes):
            v = L.FullyConnected(v, num_neurons=n, has_bias=True, weights=ws[i], name=f"wae_{tag}_fc{i}")
            if i < len(sizes) - 1:
                v = L.Relu(v, name=f"wae_{tag}_relu{i}")
        return v

    # d1 learns prior draws = 1, encoded samples (detached) = 0; d2 is a copy without an
    # optimizer, refreshed from d1 after every step, through which the encoder is trained
    # to look like the prior
    d1, d2 = weights("d1"), weights("d2", L.NoOptimizer())
    one = L.Constant(value=1.0, num_neurons=[1], name="wae_one")
    zero = L.Constant(value=0.0, num_neurons=[1], name="wae_zero")
    d_real = L.SigmoidBinaryCrossEntropy(disc(prior, d1, "d1_real"), one, name="wae_d_real")
    d_fake = L.SigmoidBinaryCrossEntropy(disc(L.StopGradient(z, name="wae_z_detached"), d1, "d1_fake"), zero,
                                         name="wae_d_fake")
    g_adv = L.SigmoidBinaryCrossEntropy(disc(z, d2, "d2_adv"), one, name="wae_g_adv")
    obj = L.ObjectiveFunction([L.LayerTerm(mse), L.LayerTerm(d_real), L.LayerTerm(d_fake),
                               L.LayerTerm(g_adv, scale=adversarial_weight)])
    copy = L.CallbackReplaceWeights(source_layers=" ".join(f"wae_d1_real_fc{i}" for i in range(len(sizes))),
                                    destination_layers=" ".join(f"wae_d2_adv_fc{i}" for i in range(len(sizes))),
                                    batch_interval=1)
    return L.Model(num_epochs, layers=list(L.traverse_layer_graph(x)), objective_function=obj,
                   metrics=[L.Metric(mse, name="reconstruction"), L.Metric(d_real, name="disc real"),
                            L.Metric(d_fake, name="disc fake"), L.Metric(g_adv, name="adversarial")],
                   callbacks=[copy])


# ------------------------------------------------------------------------ node2vec skip-gram
def construct_node2vec(num_vertices, walk_length, num_negative_samples, latent_dim=128, learning_rate=0.025,
                       embeddings="replicated", scale_decay=0.8, num_epochs=1):
    """Skip-gram with negative sampling over random walks (applications/graph/node2vec): a
    sample is ``[negative vertex ids | walk vertex ids]`` as the ``node2vec`` reader writes
    it.  Vertices of a walk attract one another with a weight that decays with their distance
    along the walk (``scale_decay`` per step), and repel the negative samples:
    positive loss = - sum_{i<j} decay^(j-i-1) log sigmoid(w_i . w_j) / normaliser,
    negative loss = - mean_{i,k} log sigmoid(-w_i . n_k).  ``embeddings="distributed"`` keeps the
    table partitioned over the ranks with sparse SGD at the owners (``DistEmbedding``)."""
    ids = L.Input(data_field="samples", name="vertex_ids")
    w = L.Weights(initializer=L.NormalInitializer(mean=0.0, standard_deviation=1.0 / latent_dim), name="embeddings")
    if embeddings == "distributed":
        emb = L.DistEmbedding(ids, weights=w, num_embeddings=num_vertices, embedding_dim=latent_dim,
                              sparse_sgd=True, learning_rate=learning_rate, name="vertex_embeddings")
    elif embeddings == "replicated":
        emb = L.Embedding(ids, weights=w, num_embeddings=num_vertices, embedding_dim=latent_dim,
                          name="vertex_embeddings")
    else:
        raise RuntimeError(f"unknown method to get embedding vectors ({embeddings})")
    sl = L.Slice(emb, axis=0, slice_points=[0, num_negative_samples, num_negative_samples + walk_length],
                 name="embedding_slice")
    neg, walk = L.Identity(sl, name="negative_embeddings"), L.Identity(sl, name="walk_embeddings")
    # all pairwise dot products of the walk: [walk, walk]; softplus(-x) = -log sigmoid(x)
    pos_dots = L.MatMul(walk, walk, transpose_b=True, name="walk_dots")
    pos_nll = L.Softplus(L.Negative(pos_dots), name="walk_nll")
    mask, norm = [], 0.0
    for i in range(walk_length):
        for j in range(walk_length):
            wgt = scale_decay ** (j - i - 1) if j > i else 0.0
            mask.append(wgt)
            norm += wgt
    pair_w = L.WeightsLayer(weights=L.Weights(initializer=L.ValueInitializer(values=[m / norm for m in mask]),
                                              optimizer=L.NoOptimizer(), name="pair_weights"),
                            dims=[walk_length, walk_length], name="pair_weight_matrix")
    pos_loss = L.Reduction(L.Multiply(pos_nll, pair_w), mode="sum", name="positive_loss")
    neg_dots = L.MatMul(walk, neg, transpose_b=True, name="negative_dots")          # [walk, negatives]
    neg_loss = L.Reduction(L.Softplus(neg_dots), mode="mean", name="negative_loss")
    return L.Model(num_epochs, layers=list(L.traverse_layer_graph(ids)),
                   objective_function=L.ObjectiveFunction([L.LayerTerm(pos_loss), L.LayerTerm(neg_loss, scale=2.0)]),
                   metrics=[L.Metric(pos_loss, name="positive loss"), L.Metric(neg_loss, name="negative loss")])


# ------------------------------------------------------------- 3-D voxel auto-encoder (MOF)
def construct_voxel_autoencoder(channels=11, size=32, base=16, latent=64, num_epochs=1):
    """Convolutional auto-encoder of voxelised crystals (metal-organic frameworks as
    ``channels`` x size^3 grids; applications/MOF/MOFae.py): three stride-2 3-D convolutions with
    batch norm down to (4 base) x (size/8)^3, a dense bottleneck, three transposed convolutions
    back; mean squared error of the reconstruction."""
    x = L.Input(data_field="samples", name="voxels")
    h = x
    for i, c in enumerate((base, 2 * base, 4 * base)):
        h = ConvolutionModule(3, c, 4, stride=2, padding=1, bias=False, name=f"mof_enc{i}")(h)
        h = L.Relu(L.BatchNormalization(h, decay=0.9, epsilon=1e-5, name=f"mof_enc{i}_bn"), name=f"mof_enc{i}_relu")
    low = size // 8
    z = FullyConnectedModule(latent, name="mof_latent")(h)
    h = L.Reshape(FullyConnectedModule(4 * base * low ** 3, activation=L.Relu, name="mof_expand")(z),
                  dims=[4 * base, low, low, low], name="mof_expand_shape")
    for i, c in enumerate((2 * base, base, channels)):
        h = ConvolutionModule(3, c, 4, stride=2, padding=1, bias=(i == 2), transpose=True, name=f"mof_dec{i}")(h)
        if i < 2:
            h = L.Relu(L.BatchNormalization(h, decay=0.9, epsilon=1e-5, name=f"mof_dec{i}_bn"), name=f"mof_dec{i}_relu")
    recon = L.Sigmoid(h, name="mof_reconstruction")
    mse = L.MeanSquaredError(recon, x, name="mof_mse")
    return L.Model(num_epochs, layers=list(L.traverse_layer_graph(x)), objective_function=L.ObjectiveFunction([mse]),
                   metrics=[L.Metric(mse, name="reconstruction error")])


# ------------------------------------------------------- image regression (HRRL ProbiesNet)
def construct_image_regressor(input_dims=(1, 300, 300), num_outputs=5, num_epochs=1):
    """Regression from single-channel images to a few physical quantities
    (applications/physics/HRRL: spectrometer images -> beam parameters): four convolution +
    pooling blocks, two dense layers; mean squared error, R^2 reported through the variance."""
    x = L.Input(data_field="samples", name="image")
    y = L.Input(data_field="responses", name="targets")
    h = x
    for i, (c, k) in enumerate(((36, 11), (64, 5), (128, 3), (128, 3))):
        h = Convolution2dModule(c, k, padding=k // 2, activation=L.Relu, name=f"reg_conv{i}")(h)
        h = L.Pooling(h, num_dims=2, has_vectors=False, pool_dims_i=2, pool_pads_i=0, pool_strides_i=2,
                      pool_mode="max", name=f"reg_pool{i}")
    h = FullyConnectedModule(480, activation=L.Relu, name="reg_fc1")(h)
    h = FullyConnectedModule(240, activation=L.Relu, name="reg_fc2")(h)
    pred = FullyConnectedModule(num_outputs, name="reg_out")(h)
    mse = L.MeanSquaredError(pred, y, name="reg_mse")
    return L.Model(num_epochs, layers=list(L.traverse_layer_graph([x, y])),
                   objective_function=L.ObjectiveFunction([mse]), metrics=[L.Metric(mse, name="mse")])
