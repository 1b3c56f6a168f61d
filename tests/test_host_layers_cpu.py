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


def test_fused_group_objects_and_their_buffer_plan_answers():
    """create_testers / create_updaters on planned groups: one head that takes the group's inputs, weights and outputs,
    followers pinned to the head's buffer, and a two-output head for the pooled and the loss forms."""
    from nnforge_b200 import host
    net = host.Net("bn BatchNorm x\nadd Add r,bn\nrelu ReLU add\npool MaxSubsampling relu win=3x3 stride=2x2\n", {"x": (8, 14, 14), "r": (8, 14, 14)})
    head, add, relu, pool = net.objects
    assert (head.role, head.kind, head.entry) == ("head", "bn_add_relu_maxpool", "nnf_bn_add_relu_maxpool_fwd")
    assert head.inputs == ["x", "r"] and head.data == ["bn"] and head.outputs == ["relu", "pool"] and head.elided == ["bn", "add"]
    assert head.get_output_count() == 2 and pool.shape == (8, 6, 6)
    assert [o.role for o in (add, relu, pool)] == ["follower"] * 3
    assert add.get_input_index_layer_can_write() == 0 and relu.get_input_index_layer_can_write() == 0 and pool.get_input_index_layer_can_write() == -1
    assert add.inputs == [] and add.outputs == []      # a follower takes and writes nothing

    net = host.Net("a PReLU x\nb ELU a\n", {"x": (4, 5, 5)})
    assert net.objects[0].kind == "bn_act" and net.objects[0].data == ["a"] and net.objects[0].outputs == ["b"]

    net = host.Net("bn BatchNorm x eps=1e-5\np PReLU bn\ne ELU p\nsm Softmax e\nl NegativeLogLikelihood sm,t,m scale=0.5\nacc Accuracy sm,t topn=3\n",
                   {"x": (8, 14, 14), "t": (8, 14, 14), "m": (1, 14, 14)}, training=True)
    head, p, e, sm, loss, acc = net.objects
    assert (head.kind, head.data, head.outputs) == ("bn_train_act", ["bn", "p"], ["e"])
    assert head.get_temporary_fixed_buffer_size() == 8 * 2 * 4 and head.get_temporary_working_fixed_buffer_size(host.FORWARD) > 0
    assert head.get_input_index_layer_can_write(host.BACKWARD_DATA_AND_WEIGHTS) == 0
    assert head.is_backward_data_and_weights_dependent_on_temporary_fixed_buffer() and not head.is_backward_data_and_weights_dependent_on_output_buffer()
    for f in (p, e):
        assert f.get_input_index_layer_can_write(host.FORWARD) == 0 and f.get_input_index_layer_can_write(host.BACKWARD_DATA) == 0
        assert not f.is_backward_data_dependent_on_input_buffer() and not f.is_backward_weights_dependent_on_input_buffer()
        assert not f.is_backward_data_dependent_on_temporary_fixed_buffer() and not f.is_backward_weights_dependent_on_temporary_per_entry_buffer()
    assert (sm.kind, sm.inputs, sm.outputs, sm.get_output_count()) == ("softmax_nll", ["e", "t", "m"], ["sm", "l"], 2)
    assert not sm.is_backward_data_dependent_on_input_buffer(0, 0) and sm.is_backward_data_dependent_on_input_buffer(0, 2)
    assert loss.role == "follower" and loss.shape == (1, 14, 14) and acc.role == "single" and acc.shape == (4, 14, 14)
    assert head.get_persistent_working_data_count() == 0 and head.get_linear_addressing_through_texture_per_entry() == []

    with pytest.raises(host.HostLayerError) as err:
        host.Net("bn BatchNorm x\n", {})
    assert "x" in str(err.value)
    # several devices share the batch: the running configuration must bring a directory for the mailboxes
    with pytest.raises(host.HostLayerError) as err:
        host.Net("bn BatchNorm x\n", {"x": (8, 4, 4)}, training=True, device_pos=0, device_count=2)
    assert "peer directory" in str(err.value)


def test_running_configuration_has_the_reference_fields():
    from nnforge_b200 import host
    rc = host.running_configuration()
    assert rc["multiprocessor_count"] > 0 and rc["smem_per_block"] > 48 * 1024 and rc["l2_cache_size"] > 0
    assert rc["compute_capability_major"] >= 1 and (rc["device_pos"], rc["device_count"]) == (0, 1)


def test_buffer_plan_of_a_fused_inference_net():
    """plan_forward_buffers: elided outputs get no buffer, a head writes over its input when nobody else reads it, freed buffers are
    taken again, network outputs stay to the end - with the objects' own get_input_index_layer_can_write answers."""
    from nnforge_b200 import host
    spec = ("bn1 BatchNorm c1\nadd1 Add bn1,skip\nrelu1 ReLU add1\npool1 MaxSubsampling relu1 win=3x3 stride=2x2\n"
            "bn2 BatchNorm pool1\ntanh2 TanH bn2\nout Sigmoid tanh2 needed\n")
    plan = host.Net(spec, {"c1": (8, 14, 14), "skip": (8, 14, 14)}).buffer_plan()
    nodes = plan["nodes"]
    assert [nodes[k]["buffer"] for k in ("bn1", "add1", "bn2", "tanh2")] == [None] * 4          # inside the fused launches
    assert nodes["relu1"]["buffer"] is not None and nodes["pool1"]["buffer"] not in (None, nodes["relu1"]["buffer"])
    assert nodes["out"]["buffer"] == nodes["pool1"]["buffer"] and nodes["out"]["in_place"] == 0  # the second group runs in place
    assert plan["buffers"] == 2 and plan["total_bytes_per_entry"] == 4 * (8 * 14 * 14 + 8 * 6 * 6)
    # the same layers with a second reader of every intermediate output: nothing fuses, nothing may be overwritten early
    unfused = ("bn1 BatchNorm c1\nadd1 Add bn1,skip\nrelu1 ReLU add1\npool1 MaxSubsampling relu1 win=3x3 stride=2x2\n"
               "tap Add bn1,add1,relu1 needed\nbn2 BatchNorm pool1\ntanh2 TanH bn2\nout Sigmoid tanh2 needed\n")
    net = host.Net(unfused, {"c1": (8, 14, 14), "skip": (8, 14, 14)})
    assert [o.role for o in net.objects[:3]] == ["single"] * 3
    plan2 = net.buffer_plan()
    n2 = plan2["nodes"]
    assert len({n2[k]["buffer"] for k in ("bn1", "add1", "relu1")}) == 3 and n2["add1"]["in_place"] is None   # bn1 is read again by the tap
    assert n2["tap"]["in_place"] == 0 and n2["tap"]["buffer"] == n2["bn1"]["buffer"]                        # the Add may write over its input 0
    assert plan2["total_bytes_per_entry"] > plan["total_bytes_per_entry"]
    with pytest.raises(host.HostLayerError):
        host.Net("bn BatchNorm x\n", {"x": (8, 4, 4)}, training=True).buffer_plan()   # the plan covers inference nets
