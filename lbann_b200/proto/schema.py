"""Field tables of the lbann_data schema (package ``lbann_data``, proto3).

One ``F(file, imports, messages, enums)`` per schema file; a message is
``M(name, fields, enums=[...], nested=[...])`` and a field is the string
``"name=number type"`` followed by ``*`` (repeated), ``?`` (explicit presence) or
``|group`` (member of the oneof ``group``).  Field names and numbers match the
prototext / binary format read by the reference executable (src/proto/*.proto), so
experiment files are interchangeable.  ``lbann_b200.proto`` turns these tables into
protobuf descriptors at import time; no protoc is involved.
"""
from ._dsl import E, F, M

FILES = [
    F('datatype', [], [
    ], enums=[E('DataType', 'DEFAULT_DATATYPE=0 FLOAT=1 DOUBLE=2 FP16=3 COMPLEX_FLOAT=4 COMPLEX_DOUBLE=5 BF16=6'), E('DeviceAllocation', 'DEFAULT_DEVICE=0 CPU=1 GPU=2')]),
    F('weights', ['datatype.proto', 'optimizers.proto'], [
        M('Weights', [
            'name=1 string', 'optimizer=2 Optimizer', 'initializer=3 Initializer',
            'datatype=4 DataType', 'sharded=5 bool', 'sharding_strategy=6 ShardingStrategy',
        ]),
        M('Initializer', [
            'constant_initializer=20 ConstantInitializer |initializer_type',
            'value_initializer=21 ValueInitializer |initializer_type',
            'numpy_initializer=22 NumpyInitializer |initializer_type',
            'uniform_initializer=23 UniformInitializer |initializer_type',
            'normal_initializer=24 NormalInitializer |initializer_type',
            'glorot_normal_initializer=25 GlorotNormalInitializer |initializer_type',
            'glorot_uniform_initializer=26 GlorotUniformInitializer |initializer_type',
            'he_normal_initializer=27 HeNormalInitializer |initializer_type',
            'he_uniform_initializer=28 HeUniformInitializer |initializer_type',
            'lecun_normal_initializer=29 LeCunNormalInitializer |initializer_type',
            'lecun_uniform_initializer=30 LeCunUniformInitializer |initializer_type',
        ], nested=[
            M('ConstantInitializer', [
                'value=1 double',
            ]),
            M('ValueInitializer', [
                'values=1 float *', 'values_d=2 double *',
            ]),
            M('NumpyInitializer', [
                'file=1 string',
            ]),
            M('UniformInitializer', [
                'min=1 double', 'max=2 double',
            ]),
            M('NormalInitializer', [
                'mean=1 double', 'standard_deviation=2 double',
            ]),
            M('GlorotNormalInitializer', [
            ]),
            M('GlorotUniformInitializer', [
            ]),
            M('HeNormalInitializer', [
            ]),
            M('HeUniformInitializer', [
            ]),
            M('LeCunNormalInitializer', [
            ]),
            M('LeCunUniformInitializer', [
            ]),
        ]),
    ], enums=[E('ShardingStrategy', 'FULL=0 GRID_ROWS=1 GRID_COLS=2')]),
    F('optimizers', [], [
        M('Optimizer', [
            'no_optimizer=1 NoOptimizer |optimizer_type', 'adagrad=2 AdaGrad |optimizer_type',
            'adam=3 Adam |optimizer_type',
            'hypergradient_adam=4 HypergradientAdam |optimizer_type',
            'rmsprop=5 RMSprop |optimizer_type', 'sgd=6 SGD |optimizer_type',
        ], nested=[
            M('NoOptimizer', [
            ]),
            M('AdaGrad', [
                'learn_rate=1 double', 'eps=2 double',
            ]),
            M('Adam', [
                'learn_rate=1 double', 'beta1=6 double', 'beta2=7 double', 'eps=8 double',
                'adamw_weight_decay=9 double',
            ]),
            M('HypergradientAdam', [
                'init_learning_rate=1 double', 'hyper_learning_rate=2 double', 'beta1=6 double',
                'beta2=7 double', 'eps=8 double',
            ]),
            M('RMSprop', [
                'learn_rate=1 double', 'decay_rate=2 double', 'eps=3 double',
            ]),
            M('SGD', [
                'learn_rate=1 double', 'momentum=2 double', 'nesterov=4 bool',
            ]),
        ]),
    ], enums=[]),
    F('operators', ['google/protobuf/any.proto', 'datatype.proto'], [
        M('Operator', [
            'input_datatype=1 DataType', 'output_datatype=2 DataType',
            'device_allocation=3 DeviceAllocation', 'parameters=4 google.protobuf.Any',
        ]),
        M('ClampOperator', [
            'min=1 double', 'max=2 double',
        ]),
        M('LogicalNotOperator', [
        ]),
        M('AbsOperator', [
        ]),
        M('NegativeOperator', [
        ]),
        M('SignOperator', [
        ]),
        M('RoundOperator', [
        ]),
        M('CeilOperator', [
        ]),
        M('FloorOperator', [
        ]),
        M('ReciprocalOperator', [
        ]),
        M('SquareOperator', [
        ]),
        M('SqrtOperator', [
        ]),
        M('RsqrtOperator', [
        ]),
        M('SafeReciprocalOperator', [
        ]),
        M('ExpOperator', [
        ]),
        M('Expm1Operator', [
        ]),
        M('LogOperator', [
        ]),
        M('Log1pOperator', [
        ]),
        M('CosOperator', [
        ]),
        M('SinOperator', [
        ]),
        M('TanOperator', [
        ]),
        M('AcosOperator', [
        ]),
        M('AsinOperator', [
        ]),
        M('AtanOperator', [
        ]),
        M('CoshOperator', [
        ]),
        M('SinhOperator', [
        ]),
        M('TanhOperator', [
        ]),
        M('AcoshOperator', [
        ]),
        M('AsinhOperator', [
        ]),
        M('AtanhOperator', [
        ]),
        M('ErfOperator', [
        ]),
        M('ErfInvOperator', [
        ]),
        M('GeluOperator', [
        ]),
        M('AddOperator', [
        ]),
        M('SubtractOperator', [
        ]),
        M('MultiplyOperator', [
        ]),
        M('DivideOperator', [
        ]),
        M('ModOperator', [
        ]),
        M('PowOperator', [
        ]),
        M('SafeDivideOperator', [
        ]),
        M('SquaredDifferenceOperator', [
        ]),
        M('MaxOperator', [
        ]),
        M('MinOperator', [
        ]),
        M('EqualOperator', [
        ]),
        M('NotEqualOperator', [
        ]),
        M('LessOperator', [
        ]),
        M('LessEqualOperator', [
        ]),
        M('GreaterOperator', [
        ]),
        M('GreaterEqualOperator', [
        ]),
        M('LogicalAndOperator', [
        ]),
        M('LogicalOrOperator', [
        ]),
        M('LogicalXorOperator', [
        ]),
        M('SelectOperator', [
            'value=1 double', 'constant_if_true=2 bool', 'constant_if_false=3 bool',
            'value_if_true=4 double', 'value_if_false=5 double', 'epsilon=6 double',
        ]),
        M('AddConstantOperator', [
            'constant=1 double',
        ]),
        M('ScaleOperator', [
            'constant=1 double',
        ]),
        M('SubtractConstantOperator', [
            'constant=1 double',
        ]),
        M('ConstantSubtractOperator', [
            'constant=1 double',
        ]),
        M('MaxConstantOperator', [
            'constant=1 double',
        ]),
        M('MinConstantOperator', [
            'constant=1 double',
        ]),
        M('NotEqualConstantOperator', [
            'constant=1 double',
        ]),
        M('EqualConstantOperator', [
            'constant=1 double',
        ]),
        M('LessEqualConstantOperator', [
            'constant=1 double',
        ]),
        M('LessConstantOperator', [
            'constant=1 double',
        ]),
        M('GreaterEqualConstantOperator', [
            'constant=1 double',
        ]),
        M('GreaterConstantOperator', [
            'constant=1 double',
        ]),
        M('LogSigmoidOperator', [
        ]),
        M('LogSoftmaxOperator', [
        ]),
        M('SeluOperator', [
        ]),
        M('SigmoidOperator', [
        ]),
        M('SoftplusOperator', [
        ]),
        M('SoftsignOperator', [
        ]),
        M('BinaryCrossEntropyOperator', [
        ]),
        M('SigmoidBinaryCrossEntropyOperator', [
        ]),
        M('BooleanAccuracyOperator', [
        ]),
        M('BooleanFalseNegativeOperator', [
        ]),
        M('BooleanFalsePositiveOperator', [
        ]),
    ], enums=[]),
    F('layers', ['google/protobuf/wrappers.proto', 'datatype.proto', 'operators.proto'], [
        M('Layer', [
            'name=1 string', 'parents=2 string *', 'children=3 string *', 'weights=4 string *',
            'device_allocation=5 string', 'datatype=6 DataType', 'hint_layer=10 string',
            'data_layout=11 string', 'parallel_strategy=12 ParallelStrategy',
            'grid_tag=13 google.protobuf.Int64Value', 'freeze=401 bool',
            'input=20 Input |layer_type', 'operator_layer=21 OperatorLayer |layer_type',
            'reshape=50 Reshape |layer_type', 'pooling=51 Pooling |layer_type',
            'concatenation=52 Concatenation |layer_type', 'slice=53 Slice |layer_type',
            'split=54 Split |layer_type', 'sum=55 Sum |layer_type',
            'cross_grid_sum_slice=56 Cross_Grid_Sum_Slice |layer_type',
            'cross_grid_sum=57 Cross_Grid_Sum |layer_type',
            'weighted_sum=58 WeightedSum |layer_type', 'unpooling=59 Unpooling |layer_type',
            'hadamard=60 Hadamard |layer_type', 'constant=61 Constant |layer_type',
            'reduction=62 Reduction |layer_type', 'evaluation=63 Evaluation |layer_type',
            'gaussian=64 Gaussian |layer_type', 'bernoulli=65 Bernoulli |layer_type',
            'uniform=66 Uniform |layer_type', 'crop=67 Crop |layer_type',
            'dummy=68 Dummy |layer_type', 'stop_gradient=69 StopGradient |layer_type',
            'in_top_k=70 InTopK |layer_type', 'sort=71 Sort |layer_type',
            'weights_layer=72 WeightsLayer |layer_type', 'tessellate=73 Tessellate |layer_type',
            'scatter=74 Scatter |layer_type', 'gather=75 Gather |layer_type',
            'batchwise_reduce_sum=76 BatchwiseReduceSum |layer_type',
            'permute=77 TensorPermute |layer_type', 'identity_zero=78 IdentityZero |layer_type',
            'multidim_reduction=79 MultiDimReduction |layer_type',
            'upsample=80 Upsample |layer_type',
            'categorical_random=406 CategoricalRandom |layer_type',
            'discrete_random=407 DiscreteRandom |layer_type',
            'fully_connected=100 FullyConnected |layer_type',
            'convolution=101 Convolution |layer_type',
            'deconvolution=102 Deconvolution |layer_type', 'embedding=103 Embedding |layer_type',
            'channelwise_scale_bias=104 ChannelwiseScaleBias |layer_type',
            'entrywise_scale_bias=105 EntrywiseScaleBias |layer_type',
            'channelwise_fully_connected=106 ChannelwiseFullyConnected |layer_type',
            'gru=107 GRU |layer_type', 'cross_entropy=120 CrossEntropy |layer_type',
            'mean_squared_error=121 MeanSquaredError |layer_type',
            'mean_absolute_error=122 MeanAbsoluteError |layer_type',
            'categorical_accuracy=123 CategoricalAccuracy |layer_type',
            'top_k_categorical_accuracy=124 TopKCategoricalAccuracy |layer_type',
            'l2_norm2=125 L2Norm2 |layer_type', 'l1_norm=126 L1Norm |layer_type',
            'matmul=140 MatMul |layer_type', 'dft_abs=141 DFTAbs |layer_type',
            'batch_normalization=160 BatchNormalization |layer_type',
            'local_response_normalization=161 LocalResponseNormalization |layer_type',
            'dropout=162 Dropout |layer_type', 'selu_dropout=163 SeluDropout |layer_type',
            'entrywise_batch_normalization=164 EntrywiseBatchNormalization |layer_type',
            'layer_norm=165 LayerNorm |layer_type', 'instance_norm=166 InstanceNorm |layer_type',
            'elu=180 Elu |layer_type', 'identity=181 Identity |layer_type',
            'leaky_relu=182 LeakyRelu |layer_type', 'log_softmax=183 LogSoftmax |layer_type',
            'relu=184 Relu |layer_type', 'softmax=185 Softmax |layer_type',
            'bilinear_resize=200 BilinearResize |layer_type', 'rotation=201 Rotation |layer_type',
            'composite_image_transformation=202 CompositeImageTransformation |layer_type',
            'cutout=203 Cutout |layer_type', 'covariance=300 Covariance |layer_type',
            'variance=301 Variance |layer_type',
            'channelwise_mean=302 ChannelwiseMean |layer_type',
            'mini_batch_index=303 MiniBatchIndex |layer_type',
            'mini_batch_size=304 MiniBatchSize |layer_type', 'argmax=305 Argmax |layer_type',
            'argmin=306 Argmin |layer_type', 'one_hot=307 OneHot |layer_type',
            'channelwise_softmax=309 ChannelwiseSoftmax |layer_type',
            'dist_embedding=311 DistEmbedding |layer_type',
            'uniform_hash=312 UniformHash |layer_type',
            'rowwise_weights_norms=313 RowwiseWeightsNorms |layer_type',
            'external=314 External |layer_type',
        ], nested=[
            M('OperatorLayer', [
                'ops=1 Operator *',
            ]),
            M('DFTAbs', [
            ]),
            M('MatMul', [
                'transpose_a=1 bool', 'transpose_b=2 bool',
            ]),
            M('Elu', [
                'alpha=1 double',
            ]),
            M('Identity', [
            ]),
            M('LeakyRelu', [
                'negative_slope=1 double',
            ]),
            M('LogSoftmax', [
            ]),
            M('Relu', [
            ]),
            M('Softmax', [
                'softmax_mode=1 string',
            ]),
            M('CrossEntropy', [
                'use_labels=1 bool',
            ]),
            M('MeanSquaredError', [
            ]),
            M('MeanAbsoluteError', [
            ]),
            M('CategoricalAccuracy', [
            ]),
            M('TopKCategoricalAccuracy', [
                'k=1 int64',
            ]),
            M('L2Norm2', [
            ]),
            M('L1Norm', [
            ]),
            M('BatchNormalization', [
                'decay=1 double', 'epsilon=4 double', 'statistics_group_size=6 int64',
                'no_bessel_correction=7 bool', 'scale_init=2 double', 'bias_init=3 double',
                'stats_aggregation=5 string',
            ]),
            M('EntrywiseBatchNormalization', [
                'decay=1 double', 'epsilon=2 double',
            ]),
            M('SeluDropout', [
                'keep_prob=2 double', 'alpha=3 double', 'scale=4 double',
            ]),
            M('LocalResponseNormalization', [
                'window_width=4 int64', 'lrn_alpha=5 double', 'lrn_beta=6 double',
                'lrn_k=7 double',
            ]),
            M('Dropout', [
                'keep_prob=2 double',
            ]),
            M('LayerNorm', [
                'epsilon=1 google.protobuf.DoubleValue', 'scale=2 bool', 'bias=3 bool',
                'start_dim=4 int64',
            ]),
            M('InstanceNorm', [
                'epsilon=1 google.protobuf.DoubleValue',
            ]),
            M('Input', [
                'data_field=1 string',
            ]),
            M('Reshape', [
                'dims=1 int64 *',
            ]),
            M('Pooling', [
                'pool_mode=1 string', 'num_dims=2 int64', 'has_vectors=3 bool',
                'pool_dims=4 int64 *', 'pool_pads=5 int64 *', 'pool_strides=6 int64 *',
                'pool_dims_i=7 int64', 'pool_pads_i=8 int64', 'pool_strides_i=9 int64',
            ]),
            M('Unpooling', [
                'num_dims=1 int64',
            ]),
            M('Concatenation', [
                'axis=1 int64',
            ]),
            M('Slice', [
                'axis=1 int64', 'slice_points=2 int64 *', 'get_slice_points_from_reader=3 string',
            ]),
            M('Split', [
            ]),
            M('Sum', [
            ]),
            M('Cross_Grid_Sum_Slice', [
            ]),
            M('Cross_Grid_Sum', [
            ]),
            M('WeightedSum', [
                'scaling_factors=1 double *',
            ]),
            M('Hadamard', [
            ]),
            M('Constant', [
                'value=1 double', 'num_neurons=2 int64 *',
            ]),
            M('Reduction', [
                'mode=1 string',
            ]),
            M('MultiDimReduction', [
                'mode=1 string', 'axes=2 uint32 *',
            ]),
            M('Evaluation', [
            ]),
            M('Gaussian', [
                'mean=1 double', 'stdev=2 double', 'neuron_dims=3 int64 *', 'training_only=4 bool',
            ]),
            M('Bernoulli', [
                'prob=1 double', 'neuron_dims=2 int64 *',
            ]),
            M('Uniform', [
                'min=1 double', 'max=2 double', 'neuron_dims=3 int64 *', 'training_only=4 bool',
            ]),
            M('Crop', [
                'dims=3 int64 *',
            ]),
            M('Dummy', [
            ]),
            M('StopGradient', [
            ]),
            M('InTopK', [
                'k=1 int64',
            ]),
            M('Sort', [
                'descending=1 bool',
            ]),
            M('WeightsLayer', [
                'dims=1 int64 *',
            ]),
            M('Tessellate', [
                'dims=1 int64 *',
            ]),
            M('Scatter', [
                'dims=1 int64 *', 'axis=2 google.protobuf.UInt64Value',
            ]),
            M('Gather', [
                'axis=1 google.protobuf.UInt64Value',
            ]),
            M('BatchwiseReduceSum', [
            ]),
            M('TensorPermute', [
                'axes=1 uint32 *',
            ]),
            M('IdentityZero', [
            ]),
            M('Upsample', [
                'upsample_mode=1 string', 'num_dims=2 int64', 'has_vectors=3 bool',
                'scale_factors=4 int64 *', 'scale_factors_i=5 int64',
            ]),
            M('CategoricalRandom', [
            ]),
            M('DiscreteRandom', [
                'values=1 double *', 'dims=2 int64 *',
            ]),
            M('FullyConnected', [
                'num_neurons=1 int64', 'has_bias=2 bool', 'transpose=3 bool',
            ]),
            M('Convolution', [
                'num_dims=1 int64', 'out_channels=2 int64', 'kernel_size=3 int64 *',
                'stride=4 int64 *', 'padding=5 int64 *', 'groups=7 google.protobuf.Int64Value',
                'has_bias=8 google.protobuf.BoolValue', 'dilation=9 int64 *',
                'conv_tensor_op_mode=14 ConvTensorOpsMode',
            ]),
            M('Deconvolution', [
                'num_dims=1 int64', 'out_channels=2 int64', 'kernel_size=3 int64 *',
                'stride=4 int64 *', 'padding=5 int64 *', 'output_padding=6 int64 *',
                'groups=7 google.protobuf.Int64Value', 'has_bias=8 google.protobuf.BoolValue',
                'dilation=9 int64 *', 'conv_tensor_op_mode=10 ConvTensorOpsMode',
            ]),
            M('Embedding', [
                'num_embeddings=1 int64', 'embedding_dim=2 int64',
                'padding_idx=3 google.protobuf.Int64Value',
            ]),
            M('ChannelwiseScaleBias', [
            ]),
            M('EntrywiseScaleBias', [
            ]),
            M('ChannelwiseFullyConnected', [
                'output_channel_dims=1 uint64 *', 'bias=2 google.protobuf.BoolValue',
                'transpose=3 google.protobuf.BoolValue',
            ]),
            M('GRU', [
                'hidden_size=1 uint64', 'num_layers=2 google.protobuf.UInt64Value',
            ]),
            M('BilinearResize', [
                'height=1 int64', 'width=2 int64',
            ]),
            M('Rotation', [
            ]),
            M('CompositeImageTransformation', [
            ]),
            M('Cutout', [
            ]),
            M('Covariance', [
                'biased=1 bool',
            ]),
            M('Variance', [
                'biased=1 bool',
            ]),
            M('ChannelwiseMean', [
            ]),
            M('MiniBatchIndex', [
            ]),
            M('MiniBatchSize', [
            ]),
            M('Argmax', [
            ]),
            M('Argmin', [
            ]),
            M('OneHot', [
                'size=1 int64',
            ]),
            M('External', [
                'filename=1 string', 'layer_name=2 string',
            ]),
            M('ChannelwiseSoftmax', [
                'dim=1 int64', 'single_dim_mode=2 bool',
            ]),
            M('DistEmbedding', [
                'num_embeddings=1 int64', 'embedding_dim=2 int64', 'sparse_sgd=3 bool',
                'learning_rate=4 double', 'barrier_in_forward_prop=5 bool',
            ]),
            M('UniformHash', [
            ]),
            M('RowwiseWeightsNorms', [
            ]),
        ]),
        M('ParallelStrategy', [
            'sample_groups=1 int64', 'sample_splits=2 int64', 'height_groups=3 int64',
            'height_splits=4 int64', 'width_groups=5 int64', 'width_splits=6 int64',
            'channel_groups=7 int64', 'channel_splits=8 int64', 'filter_groups=9 int64',
            'filter_splits=10 int64', 'replications=11 int64', 'procs_per_replica=12 int64',
            'depth_groups=13 int64', 'depth_splits=14 int64',
            'grid_tag=21 google.protobuf.Int64Value',
        ]),
        M('WeightsShape', [
            'dim=1 int64 *',
        ]),
        M('WeightsData', [
            'shape=5 WeightsShape', 'name=1 string', 'height=2 int64', 'width=3 int64',
            'data=4 float *',
        ]),
    ], enums=[E('ConvTensorOpsMode', 'DEFAULT_TENSOR_OPS=0 NO_TENSOR_OPS=1 USE_TENSOR_OPS=2 USE_TENSOR_OPS_ALLOW_CONVERSION=3'), E('Imcomm', 'DEFAULT=0 EXCLUDE=1 INCLUDE=2')]),
    F('callbacks', [], [
        M('Callback', [
            'print=1 CallbackPrint |callback_type', 'timer=2 CallbackTimer |callback_type',
            'summary=3 CallbackSummary |callback_type',
            'dump_weights=4 CallbackDumpWeights |callback_type',
            'dump_outputs=5 CallbackDumpOutputs |callback_type',
            'dump_error_signals=35 CallbackDumpErrorSignals |callback_type',
            'dump_gradients=6 CallbackDumpGradients |callback_type',
            'dump_mb_indices=7 CallbackDumpMBIndices |callback_type',
            'disp_io_stats=8 CallbackDispIOStats |callback_type',
            'save_images=10 CallbackSaveImages |callback_type',
            'debug=11 CallbackDebug |callback_type',
            'adaptive_learning_rate=12 CallbackAdaptiveLearningRate |callback_type',
            'step_learning_rate=13 CallbackStepLearningRate |callback_type',
            'set_learning_rate=55 CallbackSetLearningRate |callback_type',
            'custom_learning_rate=14 CallbackCustomLearningRate |callback_type',
            'check_small=15 CallbackCheckSmall |callback_type',
            'check_nan=16 CallbackCheckNaN |callback_type',
            'check_dataset=17 CallbackCheckDataset |callback_type',
            'hang=18 CallbackHang |callback_type',
            'drop_fixed_learning_rate=19 CallbackDropFixedLearningRate |callback_type',
            'linear_growth_learning_rate=20 CallbackLinearGrowthLearningRate |callback_type',
            'profiler=21 CallbackProfiler |callback_type',
            'step_minibatch=22 CallbackStepMinibatch |callback_type',
            'check_gradients=23 CallbackCheckGradients |callback_type',
            'ltfb=24 CallbackLTFB |callback_type', 'debug_io=25 CallbackDebugIO |callback_type',
            'minibatch_schedule=26 CallbackMinibatchSchedule |callback_type',
            'optimizerwise_adaptive_learning_rate=27 CallbackOptimizerwiseAdaptiveLearningRate |callback_type',
            'checkpoint=28 CallbackCheckpoint |callback_type',
            'save_model=29 CallbackSaveModel |callback_type',
            'poly_learning_rate=30 CallbackPolyLearningRate |callback_type',
            'replace_weights=31 CallbackReplaceWeights |callback_type',
            'gpu_memory_usage=32 CallbackGPUMemoryUsage |callback_type',
            'sync_layers=33 CallbackSyncLayers |callback_type',
            'confusion_matrix=36 CallbackConfusionMatrix |callback_type',
            'check_metric=37 CallbackCheckMetric |callback_type',
            'perturb_adam=38 CallbackPerturbAdam |callback_type',
            'perturb_dropout=39 CallbackPerturbDropout |callback_type',
            'save_topk_models=40 CallbackSaveTopKModels |callback_type',
            'mixup=41 CallbackMixup |callback_type', 'init=42 CallbackCheckInit |callback_type',
            'early_stopping=43 CallbackEarlyStopping |callback_type',
            'timeline=44 CallbackTimeline |callback_type',
            'print_model_description=45 CallbackPrintModelDescription |callback_type',
            'load_model=46 CallbackLoadModel |callback_type',
            'set_weights_value=47 CallbackSetWeightsValue |callback_type',
            'summarize_images=48 CallbackSummarizeImages |callback_type',
            'dump_model_graph=49 CallbackDumpModelGraph |callback_type',
            'perturb_learning_rate=50 CallbackPerturbLearningRate |callback_type',
            'compute_model_size=51 CallbackComputeModelSize |callback_type',
            'perturb_weights=52 CallbackPerturbWeights |callback_type',
            'export_onnx=53 CallbackExportOnnx |callback_type',
            'alternate_updates=54 CallbackAlternateUpdates |callback_type',
            'progress_bar=56 CallbackProgressBar |callback_type',
            'cosine_decay_learning_rate=57 CallbackCosineDecayLearningRate |callback_type',
            'memory_profiler=58 CallbackMemoryProfiler |callback_type',
            'clip_gradient_norm=59 CallbackClipGradientNorm |callback_type',
            'evaluate_progress=60 CallbackEvaluateProgress |callback_type',
        ], nested=[
            M('CallbackLTFB', [
                'batch_interval=1 int64', 'metric=2 string', 'weights=3 string',
                'low_score_wins=4 bool', 'communication_algorithm=5 string',
                'exchange_hyperparameters=6 bool', 'checkpoint_basedir=7 string',
            ]),
            M('CallbackStepLearningRate', [
                'weights=1 string', 'step=2 int64', 'amt=3 double',
            ]),
            M('CallbackSetLearningRate', [
                'weights=1 string', 'step=2 int64', 'val=3 double',
            ]),
            M('CallbackCustomLearningRate', [
            ]),
            M('CallbackAdaptiveLearningRate', [
                'weights=1 string', 'patience=2 int64', 'amt=3 double',
            ]),
            M('CallbackSaveImages', [
                'layers=1 string', 'image_format=2 string', 'image_prefix=3 string',
            ]),
            M('CallbackPrint', [
                'interval=1 int64', 'print_global_stat_only=2 bool',
            ]),
            M('CallbackProfiler', [
                'sync=1 bool', 'skip_init=2 bool',
            ]),
            M('CallbackTimer', [
                'skip_steps=1 int64',
            ]),
            M('CallbackSummary', [
                'batch_interval=2 int64', 'mat_interval=3 int64',
            ]),
            M('CallbackDumpWeights', [
                'directory=1 string', 'epoch_interval=2 int64', 'format=3 string',
            ]),
            M('CallbackDumpOutputs', [
                'layers=1 string', 'execution_modes=2 string', 'batch_interval=3 int64',
                'directory=4 string', 'format=5 string',
            ]),
            M('CallbackDumpErrorSignals', [
                'basename=1 string',
            ]),
            M('CallbackDumpGradients', [
                'basename=1 string', 'interval=2 int64',
            ]),
            M('CallbackDumpMBIndices', [
                'basename=1 string', 'interval=2 int64',
            ]),
            M('CallbackDispIOStats', [
                'layers=1 string',
            ]),
            M('CallbackImComm', [
                'intertrainer_comm_method=1 string', 'all_optimizers=2 bool',
            ]),
            M('CallbackDebug', [
                'phase=1 string',
            ]),
            M('CallbackDebugIO', [
                'phase=1 string', 'lvl=2 int32',
            ]),
            M('CallbackCheckSmall', [
            ]),
            M('CallbackCheckNaN', [
            ]),
            M('CallbackCheckDataset', [
            ]),
            M('CallbackHang', [
                'rank=1 int64',
            ]),
            M('CallbackDropFixedLearningRate', [
                'weights=1 string', 'drop_epoch=2 int64 *', 'amt=3 double',
            ]),
            M('CallbackLinearGrowthLearningRate', [
                'weights=1 string', 'target=2 double', 'num_epochs=3 int64', 'delay=4 int64',
            ]),
            M('CallbackPolyLearningRate', [
                'weights=1 string', 'power=2 double', 'num_epochs=3 uint64', 'max_iter=4 uint64',
                'end_lr=5 double',
            ]),
            M('CallbackCosineDecayLearningRate', [
                'weights=1 string', 'lr_max=2 double', 'lr_min=3 double', 'decay_steps=4 uint64',
                'initial_warmup_learning_rate=5 double', 'warmup_steps=6 uint64',
            ]),
            M('CallbackStepMinibatch', [
                'starting_mbsize=1 int64', 'step=2 int64', 'ramp_time=3 int64',
            ]),
            M('MinibatchScheduleStep', [
                'epoch=1 int64', 'mbsize=2 int64', 'lr=3 double', 'ramp_time=4 int64',
            ]),
            M('CallbackOptimizerwiseAdaptiveLearningRate', [
                'weights=1 string', 'scale=2 double',
            ]),
            M('CallbackMinibatchSchedule', [
                'starting_mbsize=1 int64', 'step=2 MinibatchScheduleStep *',
            ]),
            M('CallbackCheckGradients', [
                'step_size=1 double', 'verbose=2 bool', 'error_on_failure=3 bool',
                'execution_modes=4 string',
            ]),
            M('CallbackCheckMetric', [
                'metric=1 string', 'lower_bound=2 double', 'upper_bound=3 double',
                'error_on_failure=4 bool', 'execution_modes=5 string',
            ]),
            M('CallbackCheckpoint', [
                'checkpoint_dir=1 string', 'restart_dir=8 string', 'checkpoint_epochs=2 int64',
                'checkpoint_steps=3 int64', 'checkpoint_secs=4 double', 'per_rank_dir=5 string',
                'ckpt_dist_epochs=6 int64', 'ckpt_dist_steps=7 int64',
            ]),
            M('CallbackSaveModel', [
                'dir=1 string', 'extension=2 string', 'disable_save_after_training=3 bool',
            ]),
            M('CallbackLoadModel', [
                'dirs=1 string', 'extension=2 string',
            ]),
            M('CallbackReplaceWeights', [
                'source_layers=1 string', 'destination_layers=2 string', 'batch_interval=3 int64',
            ]),
            M('CallbackGPUMemoryUsage', [
            ]),
            M('CallbackSyncLayers', [
                'sync_gpus=1 bool', 'sync_mpi=2 bool', 'only_input=3 bool',
            ]),
            M('CallbackConfusionMatrix', [
                'prediction=1 string', 'label=2 string', 'prefix=3 string',
            ]),
            M('CallbackPerturbAdam', [
                'learning_rate_factor=1 float', 'beta1_factor=2 float', 'beta2_factor=3 float',
                'eps_factor=4 float', 'perturb_during_training=5 bool', 'batch_interval=6 int64',
                'weights=7 string',
            ]),
            M('CallbackPerturbDropout', [
                'keep_dropout_factor=1 float', 'layers=2 string',
            ]),
            M('CallbackSaveTopKModels', [
                'dir=1 string', 'k=2 int32', 'metric=3 string', 'ascending_ordering=4 bool',
            ]),
            M('CallbackMixup', [
                'layers=1 string', 'alpha=2 float',
            ]),
            M('CallbackCheckInit', [
            ]),
            M('CallbackEarlyStopping', [
                'patience=1 int64',
            ]),
            M('CallbackTimeline', [
                'directory=1 string',
            ]),
            M('CallbackPrintModelDescription', [
            ]),
            M('CallbackSetWeightsValue', [
                'weights=1 string', 'value=2 double', 'step=3 uint64',
            ]),
            M('CallbackSummarizeImages', [
                'selection_strategy=1 SelectionStrategy', 'image_source_layer_name=2 string',
                'epoch_interval=3 uint64',
            ], nested=[
                M('SelectionStrategy', [
                    'categorical_accuracy=1 CategoricalAccuracyStrategy |strategy_type',
                    'track_sample_ids=2 TrackSampleIDsStrategy |strategy_type',
                ], nested=[
                    M('CategoricalAccuracyStrategy', [
                        'accuracy_layer_name=1 string', 'match_type=2 MatchType',
                        'num_images_per_epoch=3 uint64',
                    ], enums=[E('MatchType', 'NOMATCH=0 MATCH=1 ALL=2')]),
                    M('TrackSampleIDsStrategy', [
                        'input_layer_name=1 string', 'num_tracked_images=2 uint64',
                    ]),
                ]),
            ]),
            M('CallbackDumpModelGraph', [
                'basename=1 string', 'print=2 bool',
            ]),
            M('CallbackPerturbLearningRate', [
                'learning_rate_factor=1 float', 'perturb_during_training=2 bool',
                'batch_interval=3 int64', 'weights=4 string',
            ]),
            M('CallbackComputeModelSize', [
                'output_name=1 string', 'batch_interval=2 int64',
            ]),
            M('CallbackPerturbWeights', [
                'upper=1 float', 'lower=2 float', 'scale=3 float', 'perturb_probability=4 float',
                'output_name=5 string', 'batch_interval=6 int64',
            ]),
            M('CallbackExportOnnx', [
                'output_filename=1 string', 'debug_string_filename=2 string',
            ]),
            M('CallbackAlternateUpdates', [
                'layers_1=1 string', 'layers_2=2 string', 'iters_1=3 int64', 'iters_2=4 int64',
            ]),
            M('CallbackProgressBar', [
                'interval=1 int64', 'newline_interval=2 int64', 'print_mem_usage=3 bool',
                'moving_average_length=4 int64', 'bar_width=5 int64', 'scientific_notation=6 bool',
            ]),
            M('CallbackMemoryProfiler', [
                'detailed_first_step=1 bool',
            ]),
            M('CallbackClipGradientNorm', [
                'weights=1 string', 'global_norm=2 bool', 'value=3 float',
            ]),
            M('CallbackEvaluateProgress', [
                'batch_interval=1 int64', 'metric=2 string',
            ]),
        ]),
    ], enums=[]),
    F('metrics', [], [
        M('Metric', [
            'layer_metric=11 LayerMetric |metric_type',
            'executable_metric=12 ExecutableMetric |metric_type',
            'python_metric=13 PythonMetric |metric_type',
        ], nested=[
            M('LayerMetric', [
                'layer=1 string', 'name=2 string', 'unit=3 string',
            ]),
            M('ExecutableMetric', [
                'name=1 string', 'filename=2 string', 'other_args=3 string',
            ]),
            M('PythonMetric', [
                'name=1 string', 'module=2 string', 'module_dir=3 string', 'function=4 string',
            ]),
        ]),
    ], enums=[]),
    F('objective_functions', [], [
        M('ObjectiveFunction', [
            'layer_term=1 LayerTerm *', 'l2_weight_regularization=2 L2WeightRegularization *',
        ], nested=[
            M('LayerTerm', [
                'scale_factor=1 double', 'layer=2 string',
            ]),
            M('L2WeightRegularization', [
                'scale_factor=1 double', 'weights=2 string *',
            ]),
        ]),
    ], enums=[]),
    F('transforms', [], [
        M('Transform', [
            'normalize=1 Normalize |transform_type',
            'sample_normalize=2 SampleNormalize |transform_type', 'scale=3 Scale |transform_type',
            'center_crop=100 CenterCrop |transform_type', 'colorize=101 Colorize |transform_type',
            'grayscale=102 Grayscale |transform_type',
            'horizontal_flip=103 HorizontalFlip |transform_type',
            'normalize_to_lbann_layout=104 NormalizeToLBANNLayout |transform_type',
            'random_affine=105 RandomAffine |transform_type',
            'random_crop=106 RandomCrop |transform_type',
            'random_resized_crop=107 RandomResizedCrop |transform_type',
            'random_resized_crop_with_fixed_aspect_ratio=108 RandomResizedCropWithFixedAspectRatio |transform_type',
            'resize=109 Resize |transform_type',
            'resized_center_crop=110 ResizedCenterCrop |transform_type',
            'to_lbann_layout=111 ToLBANNLayout |transform_type',
            'vertical_flip=112 VerticalFlip |transform_type',
            'adjust_brightness=113 AdjustBrightness |transform_type',
            'adjust_contrast=114 AdjustContrast |transform_type',
            'adjust_saturation=115 AdjustSaturation |transform_type',
            'color_jitter=116 ColorJitter |transform_type', 'cutout=117 Cutout |transform_type',
            'pad=118 Pad |transform_type',
        ], nested=[
            M('Normalize', [
                'means=1 string', 'stddevs=2 string',
            ]),
            M('SampleNormalize', [
            ]),
            M('Scale', [
                'scale=1 float',
            ]),
            M('AdjustBrightness', [
                'factor=1 float',
            ]),
            M('AdjustContrast', [
                'factor=1 float',
            ]),
            M('AdjustSaturation', [
                'factor=1 float',
            ]),
            M('CenterCrop', [
                'height=1 uint64', 'width=2 uint64',
            ]),
            M('Colorize', [
            ]),
            M('ColorJitter', [
                'min_brightness_factor=1 float', 'max_brightness_factor=2 float',
                'min_contrast_factor=3 float', 'max_contrast_factor=4 float',
                'min_saturation_factor=5 float', 'max_saturation_factor=6 float',
            ]),
            M('Cutout', [
                'num_holes=1 uint64', 'length=2 uint64',
            ]),
            M('Grayscale', [
            ]),
            M('HorizontalFlip', [
                'p=1 float',
            ]),
            M('NormalizeToLBANNLayout', [
                'means=1 string', 'stddevs=2 string',
            ]),
            M('Pad', [
                'pad=1 uint64',
            ]),
            M('RandomAffine', [
                'rotate_min=1 float', 'rotate_max=2 float', 'translate_h=3 float',
                'translate_w=4 float', 'scale_min=5 float', 'scale_max=6 float',
                'shear_min=7 float', 'shear_max=8 float',
            ]),
            M('RandomCrop', [
                'height=1 uint64', 'width=2 uint64',
            ]),
            M('RandomResizedCrop', [
                'height=1 uint64', 'width=2 uint64', 'scale_min=3 float', 'scale_max=4 float',
                'ar_min=5 float', 'ar_max=6 float',
            ]),
            M('RandomResizedCropWithFixedAspectRatio', [
                'height=1 uint64', 'width=2 uint64', 'crop_height=3 uint64', 'crop_width=4 uint64',
            ]),
            M('Resize', [
                'height=1 uint64', 'width=2 uint64',
            ]),
            M('ResizedCenterCrop', [
                'height=1 uint64', 'width=2 uint64', 'crop_height=3 uint64', 'crop_width=4 uint64',
            ]),
            M('ToLBANNLayout', [
            ]),
            M('VerticalFlip', [
                'p=1 float',
            ]),
        ]),
    ], enums=[]),
    F('reader', ['transforms.proto'], [
        M('DataReader', [
            'max_par_io_size=1 int64', 'reader=2 Reader *', 'requires_data_set_metadata=3 bool',
        ]),
        M('Reader', [
            'name=1 string', 'role=3 string', 'shuffle=4 bool', 'data_filedir=5 string',
            'data_local_filedir=50 string', 'data_filename=6 string', 'label_filename=7 string',
            'sample_list=8 string', 'validation_fraction=9 double',
            'tournament_fraction=10 double', 'absolute_sample_count=11 int64', 'first_n=200 int64',
            'fraction_of_data_to_use=12 double', 'metadata_filename=13 string',
            'gan_labelling=201 bool', 'gan_label_value=202 int32', 'num_labels=99 int32',
            'num_samples=100 int64', 'synth_dimensions=101 string',
            'synth_response_dimensions=115 string', 'separator=102 string', 'skip_cols=103 int32',
            'skip_rows=104 int32', 'has_header=105 bool', 'label_col=106 int32',
            'response_col=107 int32', 'disable_labels=108 bool', 'disable_responses=109 bool',
            'enable_labels=99108 bool', 'enable_responses=99109 bool', 'format=110 string',
            'data_file_pattern=111 string', 'num_neighbors=112 int64',
            'max_neighborhood=113 int64', 'num_image_srcs=114 int32',
            'scaling_factor_int16=116 float', 'max_files_to_load=1000 int32',
            'sample_list_per_trainer=400 bool', 'sample_list_per_model=401 bool',
            'sample_list_keep_order=402 bool', 'python=501 PythonDataReader',
            'node2vec=502 Node2VecDataReader', 'python_dataset=503 PythonDatasetReader',
            'transforms=600 Transform *', 'hdf5_key_data=700 string', 'hdf5_key_labels=701 string',
            'hdf5_key_responses=702 string', 'hdf5_hyperslab_labels=703 bool',
            'num_responses=704 int32', 'data_schema_filename=800 string',
            'experiment_schema_filename=801 string', 'synth_distribution=2001 string', 'synth_pool_size=2002 int64',
        ]),
        M('PythonDataReader', [
            'module=1 string', 'module_dir=2 string', 'sample_function=3 string',
            'num_samples_function=4 string', 'sample_dims_function=5 string',
        ]),
        M('PythonDatasetReader', [
            'dataset_path=1 string', 'module_dir=2 string', 'prefetch_factor=3 uint64',
        ]),
        M('Node2VecDataReader', [
            'graph_file=1 string', 'epoch_size=2 uint64', 'walk_length=3 uint64',
            'return_param=4 double', 'inout_param=5 double', 'num_negative_samples=6 uint64',
        ]),
        M('DataSetMetaData', [
            'schema=1 Schema', 'normalization=2 Normalization',
        ], nested=[
            M('Schema', [
                'scalar_prefix=1 string', 'image_prefix=2 string', 'input_prefix=3 string',
                'image_height=11 uint64', 'image_width=12 uint64', 'image_num_channels=13 uint64',
                'split_jag_image_channels=89 bool', 'jag_image_keys=90 string *',
                'jag_scalar_keys=91 string *', 'jag_input_keys=92 string *',
                'jag_scalar_filters=93 string *',
                'jag_scalar_prefix_filters=94 JagKeyPrefixFilter *',
                'jag_input_filters=95 string *',
                'jag_input_prefix_filters=96 JagKeyPrefixFilter *',
                'independent=97 JAGDataSlice *', 'dependent=98 JAGDataSlice *',
            ], enums=[E('JAG_Data', 'Undefined=0 JAG_Image=1 JAG_Scalar=2 JAG_Input=3')], nested=[
                M('JagKeyPrefixFilter', [
                    'key_prefix=1 string', 'min_len=2 uint32',
                ]),
                M('JAGDataSlice', [
                    'pieces=1 JAG_Data *',
                ]),
            ]),
            M('Normalization', [
                'jag_image_normalization_params=86 JagLinearNormalizationParams *',
                'jag_scalar_normalization_params=87 JagLinearNormalizationParams *',
                'jag_input_normalization_params=88 JagLinearNormalizationParams *',
            ], nested=[
                M('JagLinearNormalizationParams', [
                    'scale=1 double', 'bias=2 double',
                ]),
            ]),
        ]),
    ], enums=[]),
    F('data_coordinator', ['transforms.proto', 'datatype.proto'], [
        M('TransformDataField', [
            'data_field=1 string', 'execution_phase=2 string', 'transforms=600 Transform *',
        ]),
        M('DataCoordinator', [
            'datatype=1 DataType', 'io_buffer=2 string', 'transforms=600 TransformDataField *',
        ]),
    ], enums=[]),
    F('training_algorithm', ['google/protobuf/any.proto'], [
        M('TrainingAlgorithm', [
            'name=1 string', 'parameters=2 google.protobuf.Any',
        ]),
        M('SGD', [
            'stopping_criteria=1 TerminationCriteria', 'suppress_timer_output=489 bool',
        ], nested=[
            M('TerminationCriteria', [
                'max_batches=1 uint64 |criterion', 'max_epochs=2 uint64 |criterion',
                'max_seconds=3 double |criterion',
            ]),
        ]),
        M('LTFB', [
            'local_training_algorithm=1 TrainingAlgorithm',
            'meta_learning_strategy=2 google.protobuf.Any',
            'stopping_criteria=3 TerminationCriteria', 'suppress_timer_output=489 bool',
        ], nested=[
            M('TerminationCriteria', [
                'max_tournaments=1 uint64',
            ]),
        ]),
        M('MutationStrategy', [
            'null_mutation=1 NullMutation |strategy',
            'replace_activation=2 ReplaceActivation |strategy',
            'replace_convolution=3 ReplaceConvolution |strategy',
            'hybrid_mutation=4 HybridMutation |strategy',
        ], nested=[
            M('NullMutation', [
            ]),
            M('ReplaceActivation', [
            ]),
            M('ReplaceConvolution', [
            ]),
            M('HybridMutation', [
            ]),
        ]),
        M('RandomPairwiseExchange', [
            'metric_name_strategy_map=1 map<string,MetricStrategy>',
            'exchange_strategy=2 ExchangeStrategy', 'mutation_strategy=3 MutationStrategy',
        ], enums=[E('MetricStrategy', 'LOWER_IS_BETTER=0 HIGHER_IS_BETTER=1')], nested=[
            M('ExchangeStrategy', [
                'weights_name=1 string *', 'sendrecv_weights=2 SendRecvWeights |strategy',
                'checkpoint_binary=3 CheckpointBinary |strategy',
                'checkpoint_file=4 CheckpointFile |strategy',
            ], nested=[
                M('SendRecvWeights', [
                    'exchange_hyperparameters=1 bool',
                ]),
                M('CheckpointBinary', [
                ]),
                M('CheckpointFile', [
                    'checkpoint_dir=1 string',
                ]),
            ]),
        ]),
        M('TruncationSelectionExchange', [
            'metric_name_strategy_map=1 map<string,MetricStrategy>', 'truncation_k=2 uint64',
        ], enums=[E('MetricStrategy', 'LOWER_IS_BETTER=0 HIGHER_IS_BETTER=1')]),
        M('RegularizedEvolution', [
            'metric_name=1 string', 'metric_strategy=2 MetricStrategy',
            'mutation_strategy=3 MutationStrategy', 'sample_size=4 uint64',
        ], enums=[E('MetricStrategy', 'LOWER_IS_BETTER=0 HIGHER_IS_BETTER=1')]),
        M('KFAC', [
            'sgd=1 SGD', 'damping_act=2 string', 'damping_err=3 string', 'damping_bn_act=4 string',
            'damping_bn_err=5 string', 'kfac_use_interval=21 string',
            'damping_warmup_steps=6 uint64', 'kronecker_decay=7 double', 'print_time=8 bool',
            'print_matrix=9 bool', 'print_matrix_summary=10 bool', 'use_pi=11 bool',
            'update_intervals=12 string', 'update_interval_steps=13 uint64',
            'inverse_strategy=14 string', 'disable_layers=15 string',
            'learning_rate_factor=16 float', 'learning_rate_factor_gru=17 float',
            'compute_interval=18 int64', 'distribute_precondition_compute=19 bool',
            'use_eigen_decomposition=20 bool', 'enable_copy_errors=22 bool',
            'enable_copy_activations=23 bool',
        ]),
    ], enums=[]),
    F('trainer', ['callbacks.proto', 'training_algorithm.proto', 'data_coordinator.proto'], [
        M('Trainer', [
            'name=1 string', 'serialize_io=101 bool', 'callback=20 Callback *',
            'mini_batch_size=12 int64', 'random_init_trainers_identically=4 bool',
            'random_seed=30 int64', 'hydrogen_block_size=100 int64',
            'data_coordinator=200 DataCoordinator', 'training_algorithm=300 TrainingAlgorithm',
        ]),
    ], enums=[]),
    F('model', ['callbacks.proto', 'layers.proto', 'metrics.proto', 'objective_functions.proto', 'weights.proto'], [
        M('Model', [
            'name=3 string', 'objective_function=2 ObjectiveFunction', 'metric=5 Metric *',
            'data_layout=6 string', 'num_epochs=4 int64', 'super_steps=121 int64',
            'num_batches=122 int64', 'evaluation_frequency=54 int64',
            'subgraph_communication=13 SubGraphCommunication', 'enable_subgraph_topology=27 bool',
            'subgraph_parent_grid_resources=29 int64', 'disable_cuda=8 bool', 'layer=10 Layer *',
            'weights=11 Weights *', 'callback=20 Callback *', 'summarizer=32 Summarizer',
            'amp=60 AutomaticMixedPrecision',
        ], nested=[
            M('Summarizer', [
                'dir=1 string',
            ]),
            M('AutomaticMixedPrecision', [
                'enabled=1 bool', 'init_scale=2 double', 'growth_factor=3 double',
                'backoff_factor=4 double', 'growth_interval=5 int64',
            ]),
        ]),
    ], enums=[E('SubGraphCommunication', 'PT2PT=0 COLL=1 COLL_OPT=2')]),
    F('lbann', ['reader.proto', 'model.proto', 'optimizers.proto', 'trainer.proto', 'training_algorithm.proto'], [
        M('LbannPB', [
            'data_reader=1 DataReader', 'model=2 Model', 'optimizer=3 Optimizer',
            'data_set_metadata=5 DataSetMetaData', 'trainer=6 Trainer',
            'training_algorithm=76 TrainingAlgorithm',
        ]),
    ], enums=[]),
]
