"""Run-time counterparts of the reference proc macros (einsum validation, distributed_main, rank_sweep, module, import_model)."""
import sys, torch, pytest
from incin_b200 import macros as M, nn, io

def test_all(tmp_path):
    assert M.validate_einsum("ij,jk->ik", 2) == (["ij","jk"], "ik")
    for bad, n in (("ij,jk", 2), ("ij,jk->ik", 3), ("iJ,jk->ik", 2), ("ij,jk->iz", 2), ("ij->ii", 1), ("a->b->c", 1)):
        with pytest.raises(M.EinsumError): M.validate_einsum(bad, n)
    a, b = torch.randn(3,4), torch.randn(4,5)
    assert torch.allclose(M.einsum("ij,jk->ik", a, b), a@b, atol=1e-5)
    x, y = torch.randn(2,3,4,6), torch.randn(2,6,5)
    assert torch.allclose(M.einsum("bhmk,bkn->bnhm", x, y), torch.einsum("bhmk,bkn->bnhm", x, y), atol=1e-5)
    with pytest.raises(M.EinsumError): M.einsum("ij,jk->ik", a, torch.randn(3,5))
    with pytest.raises(M.EinsumError): M.einsum("ijk,jk->ik", a, b)
    assert M.parse_rank_args(["p", "--rank", "3", "--world-size", "8"]) == (3, 8)
    assert M.parse_rank_args(["p", "--rank", "x"]) == (0, 1)
    codes = []
    @M.distributed_main(exit_fn=codes.append)
    def main(rank, world): raise RuntimeError("boom")
    main(); assert codes == [1]
    @M.distributed_main(exit_fn=codes.append)
    def ok(rank): return rank + 10
    assert ok() == 10
    assert M.rank_sweep("names", lambda *a: a, min=1, max=3) == [("D0",), ("D0","D1"), ("D0","D1","D2")]
    assert M.rank_sweep("ranked_pairs", lambda *a: a, min=2, max=2) == [(2, ("D0",0), ("D1",1))]
    assert M.rank_sweep("conv2d", lambda *a: a, min=1, max=1) == [(2, 3, ("B0", 0))]
    assert len(M.rank_sweep("letters", lambda *a: a)) == M.max_rank()
    with pytest.raises(ValueError): M.rank_sweep("names", print, max=M.max_rank()+1)
    with M.parallel("mesh") as m:
        assert M.current_mesh() == "mesh"
        p = M.placement("Sharded(0) on M")
        assert p.kind.value == "sharded"
    assert M.current_mesh() is None
    assert M.placement("Local").kind.value == "local" and M.placement("Partial(Sum) on M").kind.value == "partial"
    with pytest.raises(ValueError): M.placement("Sharded(0)")
    assert len(M.axes("Batch", "Seq")) == 2
    @M.module
    class MLP:
        fc1: nn.Linear
        act: nn.ReLU
        fc2: nn.Linear
    nn.manual_seed(0)
    m = MLP(nn.Linear(8, 4), nn.ReLU(), nn.Linear(4, 2))
    assert [n for n, _ in m.named_layers()] == ["fc1", "act", "fc2"]
    assert set(m.state_dict_incin()) == {"fc1.weight.", "fc1.bias.", "fc2.weight.", "fc2.bias."}
    assert m(torch.randn(3, 8)).shape == (3, 2) and m.compute_stats().parameters == 8*4+4+4*2+2
    io.save_safetensors(m.state_dict_incin(), tmp_path / "m.safetensors")
    im = M.import_model(tmp_path / "m.safetensors", "Mine")
    assert type(im).__name__ == "Mine" and im.layers() == [("fc1", "Linear", (4, 8)), ("fc2", "Linear", (2, 4))]
    assert torch.equal(im.fc1.weight, m.fc1.weight)
