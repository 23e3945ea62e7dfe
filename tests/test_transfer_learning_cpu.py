"""Transfer-learning helpers: heads, selection, freezing, parameter groups, layer-wise rates, gradual unfreezing."""
import math

import pytest
import torch
import torch.nn as nn

from ml_framework_b200.modelzoo import transfer as T


def _body():
    torch.manual_seed(0)
    return nn.Sequential(nn.Linear(8, 16), nn.ReLU(), nn.Linear(16, 12), nn.ReLU(), nn.Linear(12, 10))


def test_heads_shapes_and_initialisation():
    x = torch.randn(4, 12)
    assert T.LinearHead(12, 3)(x).shape == (4, 3)
    assert T.HeadBuilder.linear_head(12, 3, include_dropout=True, dropout_rate=0.2).drop.p == 0.2
    assert T.MLPHead(12, [6, 5], 3)(x).shape == (4, 3)
    img = torch.randn(2, 6, 9, 9)
    assert T.ConvHead(6, 5, kernel_sizes=(3, 1))(img).shape == (2, 5)
    assert T.AdaptiveAvgPoolHead(6, 2, 5)(img).shape == (2, 5)
    tok = torch.randn(2, 7, 16)
    assert T.AttentionHead(16, 4, num_heads=4)(tok).shape == (2, 4)
    assert isinstance(T.HeadBuilder.create_default_head(12, 3, "attention"), T.AttentionHead)
    with pytest.raises(ValueError):
        T.HeadBuilder.create_default_head(12, 3, "tree")
    with pytest.raises(ValueError):
        T.LinearHead(0, 3)
    S = T.WeightInitializationStrategy
    assert S.KAIMING.default_parameters() == (math.sqrt(2.0), 1.0) and S.NORMAL.default_parameters() == (1.0, 0.02)
    assert S.XAVIER.is_recommended_for("tanh") and not S.XAVIER.is_recommended_for("relu") and S.KAIMING.is_recommended_for("leaky_relu")
    head = T.MLPHead(64, [64], 64)
    g = torch.Generator().manual_seed(1)
    T.initialize_weights(head, S.ORTHOGONAL, g)
    w = head.net[0].weight.detach()
    torch.testing.assert_close(w @ w.T, torch.eye(64), atol=1e-4, rtol=0)
    assert float(head.net[0].bias.detach().abs().sum()) == 0
    T.initialize_weights(head, S.TRUNCATED_NORMAL, g)
    assert float(head.net[0].weight.detach().abs().max()) <= 0.04 + 1e-6
    T.initialize_weights(head, S.NORMAL, g)
    assert 0.015 < float(head.net[0].weight.detach().std()) < 0.025


def test_head_extensions_and_adapter():
    m = _body()
    assert T.head_input_dimension(m) == 12 and "in=12 out=10" in T.head_summary(m)
    assert T.validate_head_replacement(m, T.LinearHead(12, 3)) and not T.validate_head_replacement(m, T.LinearHead(11, 3))
    old = T.replace_head(m, T.LinearHead(12, 3))
    assert isinstance(old, nn.Linear) and m(torch.randn(2, 8)).shape == (2, 3) and len(T.get_heads(m, 2)) == 2
    removed = T.remove_last_n_layers(m, 2)
    assert isinstance(removed[0], nn.ReLU) and len(m) == 3
    T.add_head(m, removed[0]); T.add_head(m, old)
    assert m(torch.randn(2, 8)).shape == (2, 10)
    with pytest.raises(T.HeadReplacementError):
        T.remove_last_n_layers(m, 9)
    with pytest.raises(T.HeadReplacementError):
        T.get_head(nn.Linear(2, 2))

    m = _body()
    a = T.HeadAdapter.adapt_pretrained(m, 4, "mlp")
    assert a.input_dim == 12 and a.num_classes == 4 and m(torch.randn(2, 8)).shape == (2, 4)
    s = T.frozen_state_summary(m)
    assert s.frozen_layers == 2 and s.unfrozen_layer_names == ["4"] and 0 < s.frozen_parameter_percentage < 100
    with pytest.raises(T.HeadAdapterError):
        a.replace_head(T.LinearHead(5, 2))
    a.replace_head(T.LinearHead(12, 2))
    assert a.num_classes == 2 and "num_classes=2" in a.summary()
    a.reset()
    assert m(torch.randn(2, 8)).shape == (2, 10) and a.num_classes == 10
    with pytest.raises(ValueError):
        a.set_number_of_classes(0)


class _Net(nn.Module):
    def __init__(self):
        super().__init__()
        self.embed = nn.Embedding(10, 8)
        self.blocks = nn.ModuleList([nn.Linear(8, 8) for _ in range(3)])
        self.act = nn.ReLU()
        self.head = nn.Linear(8, 2)

    def forward(self, ids):
        x = self.embed(ids)
        for b in self.blocks:
            x = self.act(b(x))
        return self.head(x)


def test_layer_selection_and_freezing():
    n = _Net()
    names = [k for k, _ in T.layers(n)]
    assert names == ["embed", "blocks.0", "blocks.1", "blocks.2", "act", "head"]
    L = T.LayerSelection
    assert [k for k, _ in L.by_pattern(n, r"^blocks\.[01]$")] == ["blocks.0", "blocks.1"]
    assert L.by_index(n, -1)[0] == "head" and [k for k, _ in L.by_range(n, 1, 3)] == ["blocks.0", "blocks.1"]
    assert len(L.by_type(n, nn.Linear)) == 4 and [k for k, _ in L.last_n(n, 2)] == ["act", "head"]
    assert [k for k, _ in L.first_n(n, 1)] == ["embed"] and [k for k, _ in L.by_name(n, "head", "nope")] == ["head"]
    with pytest.raises(IndexError):
        L.by_index(n, 6)
    with pytest.raises(IndexError):
        L.by_range(n, 3, 2)
    T.freeze_except_last(n, 2)
    assert [k for k, _ in T.unfrozen_layers(n)] == ["blocks.2", "head"]            # `act` has no parameters
    assert T.freeze_by_name(n, "head") == 1 and T.unfreeze_by_pattern(n, "embed") == 1
    assert [k for k, _ in T.frozen_layers(n)] == ["blocks.0", "blocks.1", "head"]
    s = T.frozen_state_summary(n)
    assert s.total_layers == 5 and s.frozen_parameters == 2 * 72 + 18 and "3/5 layers frozen" in str(s)
    T.unfreeze(n)
    assert T.frozen_state_summary(n).frozen_parameters == 0


def test_parameter_groups_builder_and_optimizer_helpers():
    n = _Net()
    T.freeze_by_pattern(n, "embed")
    b = (T.ParameterGroupBuilder()
         .new_group("frozen", 0.0).add_frozen_parameters(n)
         .new_group("early", 1e-4, 0.01).add_layers_by_pattern(r"blocks\.[01]", n)
         .new_group("late", 1e-3).add_last_n_layers(3, n).with_weight_decay(0.1).with_momentum(0.9)
         .new_group("empty", 1.0))
    groups = b.build_dictionary()
    assert set(groups) == {"frozen", "early", "late"} and b.group_count == 4
    assert groups["early"].parameter_names == ["blocks.0.weight", "blocks.0.bias", "blocks.1.weight", "blocks.1.bias"]
    assert groups["late"].parameter_count == 4 and groups["late"].momentum == 0.9 and groups["late"].total_elements == 72 + 18
    with pytest.raises(ValueError):
        b.new_group("late", 1.0)
    with pytest.raises(ValueError):
        T.ParameterGroup("g", -1.0)
    with pytest.raises(KeyError):
        T.ParameterGroupBuilder().new_group("g", 1.0).add_layer("nope", n)
    with pytest.raises(RuntimeError):
        T.ParameterGroupBuilder().add_unfrozen_parameters(n)

    T.unfreeze(n)
    opt = torch.optim.AdamW(n.parameters(), lr=1e-3)
    T.apply_parameter_groups(opt, [groups["early"], groups["late"]])
    assert [g["lr"] for g in opt.param_groups] == [1e-4, 1e-3] and opt.param_groups[1]["weight_decay"] == 0.1
    back = T.parameter_groups_of(opt, n)
    assert back[0].name == "early" and back[0].parameter_names[0] == "blocks.0.weight"
    T.set_layer_wise_lrs(opt, n, {"embed": 1e-5, "head": 1e-2}, default_lr=1e-3)
    lr_of = {id(p): g["lr"] for g in opt.param_groups for p in g["params"]}
    assert lr_of[id(n.embed.weight)] == 1e-5 and lr_of[id(n.head.bias)] == 1e-2 and lr_of[id(n.blocks[1].weight)] == 1e-3
    assert sum(len(g["params"]) for g in opt.param_groups) == len(list(n.parameters()))
    n(torch.tensor([[1, 2]])).sum().backward()
    opt.step()
    T.clear_layer_wise_lrs(opt)
    assert len(opt.param_groups) == 1 and opt.param_groups[0]["lr"] == 1e-3 and len(opt.param_groups[0]["params"]) == 9
    opt.step()                                                       # the state survived the regrouping
    d = T.create_discriminative_groups(n, 1e-3, decay=0.5).build()
    assert [round(g.learning_rate / 1e-3, 4) for g in d] == [0.0625, 0.125, 0.25, 0.5, 1.0]
    with pytest.raises(ValueError):
        T.create_discriminative_groups(n, 1e-3, multipliers=[1.0])


def test_layer_wise_scheduler_factories_schedules_and_state():
    S = T.LayerWiseLrScheduler
    s = S.create_geometric_discriminative(1e-3, 3, 0.01, 1.0)
    lrs = s.get_current_lrs()
    assert lrs["layer_0"] == pytest.approx(1e-5) and lrs["layer_1"] == pytest.approx(1e-4) and lrs["layer_2"] == pytest.approx(1e-3)
    assert s.get_parameter_learning_rate("model.layer_1.weight") == pytest.approx(1e-4)
    assert s.get_parameter_learning_rate("other") == 1e-3 and s.get_group_learning_rate(0) == 1e-3
    g = S.create_gradual_unfreezing(1e-3, 3, 1e-5, 1e-3)
    assert g.get_parameter_learning_rate("layer_1") == pytest.approx((1e-5 + 1e-3) / 2)
    tri = S.create_triangular(1e-3, 1e-4, 1e-2, cycle_steps=100)
    assert tri.get_parameter_learning_rate("w") == pytest.approx(1e-4)
    tri.step_count = 25
    assert tri.get_parameter_learning_rate("w") == pytest.approx((1e-4 + 1e-2) / 2)
    tri.step_count = 500
    assert tri.get_parameter_learning_rate("w") == pytest.approx(1e-2)
    wc = S.create_warmup_cosine(1e-3, 5e-3, 10, 110)
    wc.step_count = 5
    assert wc.get_parameter_learning_rate("warmup.w") == pytest.approx(3e-3)
    wc.step_count = 110
    assert wc.get_parameter_learning_rate("annealing.w") == pytest.approx(1e-5)
    st = S(1.0)
    st.set_layer_schedule("a", T.ScheduleType.STEP, 2.0, 0.5, 10)
    st.set_layer_schedule("b", T.ScheduleType.CONSTANT, 3.0, 9.0, 10)
    st.set_multiplier("c", 0.25)
    assert st.scheduled_layer_count == 3
    vals = []
    for _ in range(10):
        vals.append(st.get_parameter_learning_rate("a"))
        st.step()
    assert vals[:5] == [2.0] * 5 and vals[5:] == [0.5] * 5 and st.get_parameter_learning_rate("b") == 3.0
    other = S(5.0)
    other.load_state_dict(st.state_dict())
    assert other.get_current_lrs() == st.get_current_lrs() and other.step_count == 10
    # applied to an optimiser through named groups
    n = _Net()
    opt = torch.optim.SGD(n.parameters(), lr=1.0)
    T.apply_parameter_groups(opt, T.create_discriminative_groups(n, 1.0))
    sched = S.create_discriminative(1.0, [0.1, 0.2, 0.3, 0.4, 0.5])
    assert sched.apply(opt) == pytest.approx([0.1, 0.2, 0.3, 0.4, 0.5])
    for bad in (lambda: S(0.0), lambda: S.create_discriminative(1.0, []), lambda: S.create_triangular(1.0, 2.0, 1.0),
                lambda: S.create_warmup_cosine(1.0, 1.0, 10, 10), lambda: st.set_multiplier("x", -1.0)):
        with pytest.raises(ValueError):
            bad()


def test_gradual_unfreezing_stages():
    n = _Net()
    seen = []
    g = T.GradualUnfreezingScheduler.create_evenly_distributed(n, 4)
    g.on_unfreeze_stage.append(lambda s, total: seen.append((s, total)))
    assert g.unfreeze_thresholds == [0.25, 0.5, 0.75, 1.0]
    assert not g.update_unfreezing(0.1) and T.frozen_state_summary(n).unfrozen_layers == 0
    assert g.update_unfreezing(0.3) and [k for k, _ in T.unfrozen_layers(n)] == ["head"]
    assert not g.update_unfreezing(0.4)
    assert g.update_unfreezing(0.8) and g.current_stage == 2 and len(T.unfrozen_layers(n)) == 3   # jumps over a stage
    assert g.advance_to_next_stage() and not g.advance_to_next_stage() and seen == [(0, 4), (2, 4), (3, 4)]
    g.set_stage(0)
    assert [k for k, _ in T.unfrozen_layers(n)] == ["head"] and g.unfrozen_layer_count(0) == 1 and g.unfrozen_layer_count(-1) == 0
    assert "stage 1/4" in g.state_summary()
    g.reset()
    assert g.current_stage == -1 and not T.unfrozen_layers(n)
    for bad in ([], [0.5, 0.2], [1.5]):
        with pytest.raises(ValueError):
            T.GradualUnfreezingScheduler(n, bad)
    with pytest.raises(ValueError):
        g.update_unfreezing(1.5)
    with pytest.raises(ValueError):
        g.set_stage(4)
