"""GPU test: a forward + backward pair captured into a CUDA graph and replayed.  Everything the operators enqueue is
stream work (a memset node and kernels; tensor maps are encoded on the host at capture time), so a training loop can
put them into a graph; the backward's work counter and status word are reset by the captured memset at every
replay."""
import pytest
import torch

from hopper_jeni_b200 import ops

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("D,causal,B,Hq,Hkv,S", [(64, False, 4, 6, 2, 4096), (128, True, 4, 8, 4, 2048)])
def test_forward_backward_replay_from_a_cuda_graph(gqa_lib, D, causal, B, Hq, Hkv, S):
    # 256 work items each: more than SMs, so the persistent blocks of the backward claim items from the counter
    gen = torch.Generator(device="cuda").manual_seed(31)

    def fresh(h):
        return torch.randn(B, h, S, D, generator=gen, device="cuda").bfloat16()

    q, k, v, do = fresh(Hq), fresh(Hkv), fresh(Hkv), fresh(Hq)
    o, lse = torch.empty_like(q), torch.empty(B, Hq, S, dtype=torch.float32, device="cuda")
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    ws = torch.empty(ops.bwd_workspace_bytes(B, Hq, Hkv, S, D, causal), dtype=torch.uint8, device="cuda")

    def step():
        ops.gqa_forward(q, k, v, causal=causal, out=o, lse=lse)
        ops.gqa_backward(q, k, v, o, do, lse, causal=causal, workspace=ws, dq=dq, dk=dk, dv=dv)

    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):      # warm-up outside the capture (first-use look-ups, module loading)
        step()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        step()
    for trial in range(3):
        for t, h in ((q, Hq), (k, Hkv), (v, Hkv), (do, Hq)):
            t.copy_(fresh(h))
        for t in (o, dq, dk, dv):
            t.fill_(float("nan"))
        graph.replay()
        torch.cuda.synchronize()
        ops.check_status(ws)
        ops.check_status()
        got = [t.clone() for t in (o, lse, dq, dk, dv)]
        step()                          # the same inputs, eagerly
        torch.cuda.synchronize()
        assert torch.equal(got[0], o) and torch.equal(got[1], lse), trial
        assert torch.equal(got[3], dk) and torch.equal(got[4], dv), trial
        assert torch.isfinite(got[2].float()).all()
        rel = (got[2].float() - dq.float()).norm() / dq.float().norm()
        assert rel < 2e-3, (trial, float(rel))  # dQ: same sums, order of the fp32 reductions varies
