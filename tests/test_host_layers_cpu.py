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
