"""``lbann.models``: model zoo (LeNet, AlexNet, ResNet, CosmoFlow, U-Net3D, Transformer / GPT, RoBERTa,
sub-graph Transformer) and the application models (auto-encoders, VAE, GAN, DenseNet, character GRU,
dense-graph GCN, siamese patches, CANDLE combo, JAG WAE)."""
from .lenet import LeNet  # noqa: F401
from .cosmoflow import CosmoFlow, construct_cosmoflow_model  # noqa: F401
from .resnet import (AlexNet, ResNet, ResNet18, ResNet34, ResNet50, ResNet101, ResNet152,  # noqa: F401
                     construct_classifier)
from .transformer import (GPT, LayerNorm, Transformer, TransformerDecoderLayer,  # noqa: F401
                          TransformerEncoderLayer, causal_mask, construct_gpt_model)
from .unet3d import UNet3D, construct_unet3d_model  # noqa: F401
from .roberta import RoBERTa, RobertaConfig  # noqa: F401
from . import subgraph  # noqa: F401
from . import applications  # noqa: F401
from .applications import (construct_autoencoder, construct_candle_combo, construct_char_rnn,  # noqa: F401
                           construct_dense_gcn, construct_densenet, construct_gan, construct_jag_wae,
                           construct_image_regressor, construct_node2vec, construct_siamese, construct_vae,
                           construct_voxel_autoencoder)
