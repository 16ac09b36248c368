import pickle

import numpy as np
import pytest
import torch

from verl_b200.protocol import (DataProto, DataProtoFuture, Jagged, pad_dataproto_to_divisor, unpad_dataproto, union_tensor_dict)


def make(n=6):
    return DataProto.from_dict(tensors={"a": torch.arange(n * 2).reshape(n, 2), "b": torch.arange(n).float()},
                               non_tensors={"s": np.array([f"x{i}" for i in range(n)], dtype=object)}, meta_info={"k": 1})


def test_basic_len_and_index():
    d = make()
    assert len(d) == 6
    item = d[2]
    assert item.batch["a"].tolist() == [4, 5] and item.non_tensor_batch["s"] == "x2"
    sl = d[1:4]
    assert len(sl) == 3 and sl.non_tensor_batch["s"].tolist() == ["x1", "x2", "x3"]
    sel = d[[0, 5]]
    assert sel.batch["b"].tolist() == [0.0, 5.0]
    mask = torch.tensor([True, False, True, False, False, False])
    assert len(d[mask]) == 2


def test_chunk_concat_roundtrip():
    d = make(8)
    parts = d.chunk(4)
    assert [len(p) for p in parts] == [2, 2, 2, 2]
    back = DataProto.concat(parts)
    assert torch.equal(back.batch["a"], d.batch["a"]) and back.non_tensor_batch["s"].tolist() == d.non_tensor_batch["s"].tolist()
    with pytest.raises(AssertionError):
        make(7).chunk(2)


def test_concat_merges_metrics():
    a, b = make(2), make(2)
    a.meta_info["metrics"] = {"loss": [1.0]}
    b.meta_info["metrics"] = {"loss": [3.0], "kl": 0.5}
    c = DataProto.concat([a, b])
    assert c.meta_info["metrics"]["loss"] == [1.0, 3.0] and c.meta_info["metrics"]["kl"] == [0.5]


def test_repeat_interleave_and_tile():
    d = make(3)
    r = d.repeat(2, interleave=True)
    assert r.batch["b"].tolist() == [0, 0, 1, 1, 2, 2]
    r2 = d.repeat(2, interleave=False)
    assert r2.batch["b"].tolist() == [0, 1, 2, 0, 1, 2]
    assert r.non_tensor_batch["s"].tolist() == ["x0", "x0", "x1", "x1", "x2", "x2"]


def test_union_and_conflict():
    d = make(4)
    e = DataProto.from_dict(tensors={"c": torch.ones(4)})
    d.union(e)
    assert "c" in d.batch
    bad = DataProto.from_dict(tensors={"b": torch.zeros(4)})
    with pytest.raises(AssertionError):
        d.union(bad)


def test_select_pop_rename():
    d = make(4)
    s = d.select(batch_keys=["a"])
    assert list(s.batch.keys()) == ["a"]
    p = d.pop(batch_keys=["b"], non_tensor_batch_keys=["s"])
    assert "b" not in d.batch and "b" in p.batch and "s" in p.non_tensor_batch
    d.rename("a", "z")
    assert "z" in d.batch


def test_padding_helpers():
    d = make(5)
    padded, pad = pad_dataproto_to_divisor(d, 4)
    assert len(padded) == 8 and pad == 3
    assert torch.equal(unpad_dataproto(padded, pad).batch["a"], d.batch["a"])
    same, p0 = pad_dataproto_to_divisor(make(4), 4)
    assert p0 == 0 and len(same) == 4


def test_auto_padding_chunk():
    d = DataProto.from_dict(tensors={"a": torch.arange(5)}, auto_padding=True)
    parts = d.chunk(2)
    assert sum(len(p) for p in parts) == 5


def test_reorder_and_iterator():
    d = make(4)
    d.reorder(torch.tensor([3, 2, 1, 0]))
    assert d.batch["b"].tolist() == [3, 2, 1, 0] and d.non_tensor_batch["s"][0] == "x3"
    it = d.make_iterator(2, epochs=2, seed=0)
    assert sum(len(x) for x in it) == 8


@pytest.mark.parametrize("method", ["torch", "numpy"])
def test_pickle_roundtrip(monkeypatch, method):
    monkeypatch.setenv("VERL_DATAPROTO_SERIALIZATION_METHOD", method)
    d = make(3)
    d.batch["h"] = torch.randn(3, 2).bfloat16()
    d.batch["j"] = Jagged.from_list([torch.arange(2), torch.arange(3), torch.arange(1)])
    e = pickle.loads(pickle.dumps(d))
    assert torch.equal(e.batch["a"], d.batch["a"]) and torch.equal(e.batch["h"], d.batch["h"])
    assert e.batch["j"].lengths.tolist() == [2, 3, 1] and e.meta_info == {"k": 1}


def test_jagged_ops():
    j = Jagged.from_list([torch.arange(3), torch.arange(1), torch.arange(2)])
    assert j.to_padded(-1).tolist() == [[0, 1, 2], [0, -1, -1], [0, 1, -1]]
    assert j.index(torch.tensor([2, 0])).lengths.tolist() == [2, 3]
    assert j.slice(1, 3).values.tolist() == [0, 0, 1]
    padded = torch.tensor([[0, 0, 5, 6], [0, 7, 8, 9]])
    assert Jagged.from_padded(padded, torch.tensor([2, 3]), left_pad=True).values.tolist() == [5, 6, 7, 8, 9]


def test_future_get():
    class F:
        def __init__(self, v):
            self.v = v

        def result(self):
            return self.v

    fut = DataProtoFuture.concat([F(make(2)), F(make(2))])
    parts = fut.chunk(2)
    assert len(parts[1].get()) == 2 and len(fut.get()) == 4


def test_union_tensor_dict_mismatch_batch():
    from verl_b200.protocol import TensorBatch

    with pytest.raises(AssertionError):
        union_tensor_dict(TensorBatch({"a": torch.zeros(2)}), TensorBatch({"b": torch.zeros(3)}))


def test_tensordict_helper_surface():
    """The helper functions the engine path uses on batches: shared vs per-sample non-tensor data, ragged rows, key access across
    the three places a value can live, concatenation, union, equality and the row-dict constructor."""
    import numpy as np
    import pytest
    import torch

    from verl_b200.protocol import Jagged
    from verl_b200.utils import tensordict_utils as tu

    rows = [{"ids": torch.arange(3), "score": torch.tensor(0.5), "uid": "a", "tools": [1, 2]},
            {"ids": torch.arange(5), "score": torch.tensor(1.5), "uid": "b", "tools": []}]
    d = tu.list_of_dict_to_tensordict(rows)
    assert isinstance(d.batch["ids"], Jagged) and d.batch["score"].tolist() == [0.5, 1.5] and tu.get(d, "uid") == ["a", "b"]
    tu.assign_non_tensor_data(d, "temperature", 0.7)
    tu.assign_non_tensor_stack(d, "extra", [{"k": 1}, {"k": 2}])
    with pytest.raises(ValueError):
        tu.assign_non_tensor_stack(d, "bad", [1])
    assert tu.get(d, "temperature") == 0.7 and tu.get(d, "extra")[1] == {"k": 2} and tu.get(d, "missing", 3) == 3
    assert tu.unwrap_non_tensor_data(np.array(4)) == 4 and tu.unwrap_non_tensor_data(d.non_tensor_batch["tools"]) == [[1, 2], []]
    sub = tu.get_keys(d, ["score", "uid", "temperature"])
    assert set(sub.batch.keys()) == {"score"} and set(sub.non_tensor_batch) == {"uid"} and sub.meta_info == {"temperature": 0.7}
    with pytest.raises(KeyError):
        tu.get_keys(d, ["nope"])
    both = tu.concat_tensordict([d, d])
    assert len(both) == 4 and [len(r) for r in both.batch["ids"].unbind()] == [3, 5, 3, 5] and tu.get(both, "uid") == ["a", "b", "a", "b"]
    tu.assert_tensordict_eq(both[:2], d)
    with pytest.raises(AssertionError, match="differs"):
        other = tu.list_of_dict_to_tensordict(rows)
        other.batch["score"] = torch.tensor([0.5, 9.0])
        tu.assign_non_tensor_data(other, "temperature", 0.7)
        tu.assign_non_tensor_stack(other, "extra", [{"k": 1}, {"k": 2}])
        tu.assert_tensordict_eq(other, d)
    u = tu.union_tensor_dict(tu.get_keys(d, ["score"]), tu.get_tensordict({"adv": torch.ones(2, 4)}))
    assert set(u.batch.keys()) == {"score", "adv"}
    popped = tu.pop_keys(d, ["score", "temperature"])
    assert "score" not in d.batch.keys() and "temperature" not in d.meta_info and popped.batch["score"].shape == (2,)
    assert tu.pop(d, "uid") == ["a", "b"] and tu.pop(d, "uid", None) is None
    j = tu.concat_nested_tensors([tu.nested_tensor_from_tensor_list([torch.ones(2), torch.ones(1)]), tu.nested_tensor_from_tensor_list([torch.ones(4)])])
    assert j.offsets.tolist() == [0, 2, 3, 7]
    shared = tu.concat_tensordict_with_none_bsz([tu.get_tensordict({}, {"a": 1}), tu.get_tensordict({}, {"a": 1, "b": 2})])
    assert shared.meta_info == {"a": 1, "b": 2}
    with pytest.raises(ValueError, match="differs"):
        tu.concat_tensordict_with_none_bsz([tu.get_tensordict({}, {"a": 1}), tu.get_tensordict({}, {"a": 2})])
    import pickle

    p = tu.get_tensordict({"position_ids": [torch.zeros(4, 3), torch.zeros(6, 3)]})          # ragged multimodal positions, one [L_i, 3] per sample
    back = tu.maybe_fix_3d_position_ids(pickle.loads(pickle.dumps(p)))
    assert [tuple(r.shape) for r in back.batch["position_ids"].unbind()] == [(4, 3), (6, 3)]
    t = tu.get_tensordict({"x": torch.arange(12).reshape(2, 6).t()[:, :2].t()})
    assert tu.contiguous(t).batch["x"].is_contiguous()
