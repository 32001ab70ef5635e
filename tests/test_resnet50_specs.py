"""Layer list of the ResNet-50-shaped stack (host logic, no GPU)."""
from shflbw_sparse_nn_b200.resnet50 import layer_specs


def test_layer_list_matches_the_reference_sweep_shapes():
    """The distinct (Ho, C, F, R, stride) of the stack are the 22 shapes of the reference's sweep
    list (scripts/benchmark/conv.block_sparse.sh:5-27), 52 layers in all."""
    specs = layer_specs(56)
    assert len(specs) == 52
    shapes = {(s.Ho, s.C, s.F, s.R, s.stride) for s in specs}
    want = {(56, 64, 64, 1, 1), (56, 256, 64, 1, 1), (56, 64, 64, 3, 1), (56, 64, 256, 1, 1), (56, 256, 128, 1, 1),
            (28, 512, 128, 1, 1), (28, 128, 128, 3, 2), (28, 128, 128, 3, 1), (28, 128, 512, 1, 1), (28, 256, 512, 1, 2),
            (28, 512, 256, 1, 1), (14, 1024, 256, 1, 1), (14, 256, 256, 3, 2), (14, 256, 256, 3, 1), (14, 256, 1024, 1, 1),
            (14, 512, 1024, 1, 2), (14, 1024, 512, 1, 1), (7, 2048, 512, 1, 1), (7, 512, 512, 3, 2), (7, 512, 512, 3, 1),
            (7, 512, 2048, 1, 1), (7, 1024, 2048, 1, 2)}
    assert shapes == want


def test_data_flow_indices_are_consistent():
    specs = layer_specs(56)
    for i, s in enumerate(specs):
        assert -1 <= s.src < i
        if s.src >= 0:
            assert specs[s.src].F == s.C and specs[s.src].Ho == s.Hin and specs[s.src].consumers_R == s.R
        if s.residual is not None and s.residual >= 0:
            r = specs[s.residual]
            assert r.residual is not None or r.name.endswith("proj")
            assert r.F == s.F and r.Ho == s.Ho and r.consumers_R == s.consumers_R
