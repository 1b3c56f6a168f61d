"""C++ host-side layer objects: construction through the factory by nnForge type name, buffer-plan
answers and error behaviour. No kernel is launched here."""
import pytest


def test_factory_knows_its_type_names_and_rejects_others():
    from nnforge_b200 import host
    for name in ("BatchNorm", "ReLU", "PReLU", "ELU", "TanH", "Sigmoid", "Softmax", "Add"):
        assert host.Tester(name, 8, 5, 5).h
        assert host.Updater(name, 8, 5, 5).h
    assert host.Tester("MaxSubsampling", 8, 9, 9, pool=[3, 3, 2, 2, 0, 0, 0]).h
    assert host.Tester("NegativeLogLikelihood", 8, 5, 5, params=[1.0], input_count=2).h
    assert host.Tester("AverageSubsampling", 8, 6, 6, pool=[3, 2, 0, 0, 0, 0, 0]).h
    with pytest.raises(host.HostLayerError) as e:
        host.Tester("AverageSubsampling", 8, 7, 7, pool=[2, 2, 0, 0, 0, 0, 0])
    assert "divisible" in str(e.value)
    assert host.Tester("Accuracy", 8, 5, 5, params=[3], input_count=2).h
    assert host.Updater("Accuracy", 8, 5, 5, params=[1], input_count=3, with_backward=False).h
    loss = host.Updater("NegativeLogLikelihood", 8, 5, 5, params=[1.0], input_count=3)
    assert loss.is_backward_data_dependent_on_input_buffer() and not loss.is_backward_data_dependent_on_output_buffer()
    with pytest.raises(host.HostLayerError) as e:
        host.Tester("Convolution", 8, 5, 5)
    assert "Convolution" in str(e.value)


def test_buffer_plan_answers_follow_the_reference_layers():
    from nnforge_b200 import host
    bn = host.Updater("BatchNorm", 16, 7, 7, params=[1e-5])
    assert bn.get_temporary_fixed_buffer_size() == 16 * 2 * 4          # mean + inverse std-dev, as the stock updater
    assert bn.get_input_index_layer_can_write(host.BACKWARD_DATA_AND_WEIGHTS) == 0
    assert bn.get_input_index_layer_can_write(host.FORWARD) == -1
    assert bn.get_temporary_working_fixed_buffer_size(host.FORWARD) > 16 * 2 * 4
    relu = host.Updater("ReLU", 4, 3, 3, params=[0.0])
    assert relu.is_backward_data_dependent_on_input_buffer() and not relu.is_backward_data_dependent_on_output_buffer()
    assert relu.get_temporary_per_entry_buffer_size() == 0               # no bit-mask buffer: the gate is read from the input
    elu = host.Updater("ELU", 4, 3, 3)
    assert elu.is_backward_data_dependent_on_output_buffer() and not elu.is_backward_data_dependent_on_input_buffer()
    sm = host.Updater("Softmax", 10, 1, 1)
    assert sm.get_input_index_layer_can_write(host.BACKWARD_DATA) == 0 and sm.is_backward_data_dependent_on_output_buffer()
    pool = host.Updater("MaxSubsampling", 4, 9, 7, pool=[3, 3, 2, 2, 0, 0, 0])
    assert pool.get_temporary_per_entry_buffer_size() == 4 * 4 * 3 * 4   # 4 maps x (4 x 3) outputs x uint32 offsets
    assert not pool.is_backward_data_dependent_on_input_buffer() and not pool.is_backward_data_dependent_on_output_buffer()
    assert host.Updater("MaxSubsampling", 4, 9, 7, pool=[3, 3, 2, 2, 0, 0, 0], with_backward=False).get_temporary_per_entry_buffer_size() == 0


def test_empty_output_is_an_error_like_in_the_reference():
    from nnforge_b200 import host
    with pytest.raises(host.HostLayerError) as e:
        host.Tester("MaxSubsampling", 4, 2, 2, pool=[3, 3, 2, 2, 0, 0, 0])
    assert "0 output size" in str(e.value)


RESNET_TAIL = """
conv1 Convolution data
bn1 BatchNorm conv1
relu1 ReLU bn1
conv2 Convolution relu1
bn2 BatchNorm conv2
add Add bn2,relu1
relu2 ReLU add
pool MaxSubsampling relu2 win=3x3
conv3 Convolution pool
bn3 BatchNorm conv3
add3 Add bn3,pool
relu3 ReLU add3
gap AverageSubsampling relu3 win=7x7
fc Convolution gap
sm Softmax fc
loss NegativeLogLikelihood sm,labels
acc Accuracy sm,labels
"""


def _groups(spec, training=False):
    from nnforge_b200 import host
    return {g["members"][0]: g for g in host.plan_fusion(spec, training)}


def test_fusion_peephole_on_a_residual_tail():
    g = _groups(RESNET_TAIL)
    assert g["bn1"]["kind"] == "bn_act" and g["bn1"]["members"] == ["bn1", "relu1"] and g["bn1"]["elided"] == ["bn1"]
    # relu1 feeds conv2 and the Add: its output exists, and it is the Add's residual
    blk = g["bn2"]
    assert blk["kind"] == "bn_add_relu_maxpool" and blk["entry_point"] == "nnf_bn_add_relu_maxpool_fwd"
    assert blk["members"] == ["bn2", "add", "relu2", "pool"] and blk["residual"] == "relu1"
    assert blk["elided"] == ["bn2", "add"]                       # z = relu2 is written by the fused kernel
    tail = g["bn3"]
    assert tail["kind"] == "bn_add_relu_avgpool" and tail["members"] == ["bn3", "add3", "relu3", "gap"] and tail["residual"] == "pool"
    sm = g["sm"]
    assert sm["kind"] == "softmax_nll" and sm["members"] == ["sm", "loss"] and sm["elided"] == []   # the probabilities stay for Accuracy
    assert g["acc"]["kind"] == "single" and g["conv1"]["kind"] == "single"
    every = sorted(m for grp in g.values() for m in grp["members"])
    assert every == sorted(line.split()[0] for line in RESNET_TAIL.strip().splitlines())           # every layer in exactly one group


def test_fusion_peephole_respects_other_readers_and_parameters():
    # the batch-norm output is read twice: nothing may swallow it
    g = _groups("bn BatchNorm x\nrelu ReLU bn\nside Convolution bn\n")
    assert g["bn"]["kind"] == "single" and g["relu"]["kind"] == "single"
    # an output that is needed elsewhere stays
    g = _groups("bn BatchNorm x needed\nrelu ReLU bn\n")
    assert g["bn"]["kind"] == "single"
    # two activations fuse, a third starts a new group; at most one PReLU per chain
    g = _groups("bn BatchNorm x\na PReLU bn\nb ELU a\nc TanH b\n")
    assert g["bn"]["members"] == ["bn", "a", "b"] and g["c"]["kind"] == "single"
    g = _groups("bn BatchNorm x\na PReLU bn\nb PReLU a\n")
    assert g["bn"]["members"] == ["bn", "a"] and g["b"]["kind"] == "single"
    # Add with alpha != 1 cannot take the pooled form but still fuses with its activation
    g = _groups("bn BatchNorm x\nadd Add bn,r alpha=0.5\nrelu ReLU add\npool MaxSubsampling relu win=2x2\n")
    assert g["bn"]["kind"] == "bn_act" and g["bn"]["members"] == ["bn", "add", "relu"] and g["pool"]["kind"] == "single"
    # feature-map subsampling is not a 2-D window
    g = _groups("bn BatchNorm x\nrelu ReLU bn\npool MaxSubsampling relu win=2x2 fm=2\n")
    assert g["bn"]["kind"] == "bn_act" and g["pool"]["kind"] == "single"
    # a residual that is produced after the batch norm cannot be read by a kernel that runs at the batch norm's place
    g = _groups("bn BatchNorm x\nlate Convolution y\nadd Add bn,late\n")
    assert g["bn"]["kind"] == "single" and g["add"]["kind"] == "single"


def test_fusion_peephole_training_patterns():
    spec = "bn BatchNorm x\na PReLU bn\nb ELU a\nsm Softmax b\nloss NegativeLogLikelihood sm,t,mask\n"
    g = _groups(spec, training=True)
    assert g["bn"]["kind"] == "bn_train_act" and g["bn"]["entry_point"] == "nnf_bn_train_fwd" and g["bn"]["elided"] == ["bn", "a"]
    assert g["sm"]["kind"] == "softmax_nll"
    # the frozen-statistics pooled form is an inference pattern only
    g = _groups("bn BatchNorm x\nadd Add bn,r\nrelu ReLU add\npool MaxSubsampling relu win=3x3\n", training=True)
    assert g["bn"]["kind"] == "single"
    from nnforge_b200 import host
    with pytest.raises(host.HostLayerError):
        host.plan_fusion("b ReLU a\na BatchNorm x\n")    # not in execution order
