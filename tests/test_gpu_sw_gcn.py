"""torch.ops.sw_gcn on CUDA tensors: the layers of the reference's GCN scripts, written exactly as they call the
operators (binding-project/gcn-e2e-training/FusedGCNLayer.py:8-42, FusedGCNModule.py:7-18), against dense torch."""
import pytest

from tests import common
from tile_fusion_b200 import synth

pytestmark = pytest.mark.gpu


def _layers(torch):
    import tile_fusion_b200.sw_gcn  # noqa: F401  (registers torch.ops.sw_gcn)

    class FusedGCNLayer(torch.nn.Module):  # as FusedGCNLayer.py:8-42
        def __init__(self, feat_dim, embed_dim, m_tile_size, adj, schedule, num_threads):
            super().__init__()
            self.weight = torch.nn.Parameter(torch.empty(embed_dim, feat_dim, device="cuda"))
            torch.nn.init.xavier_uniform_(self.weight)
            self.adj, self.schedule, self.num_threads = adj, schedule, num_threads
            self.forward_fn = torch.ops.sw_gcn.fusedGeMMSpMM_vt_ro
            level_ptr, mix_ptr = self.schedule[0], self.schedule[1]
            self.max_tile_size = 0
            for x in range(level_ptr[0], level_ptr[1]):
                self.max_tile_size = max(self.max_tile_size, int(mix_ptr[x * 2 + 2] - mix_ptr[x * 2]))

        def forward(self, x):
            return self.forward_fn(self.adj, x, self.weight, self.schedule, self.num_threads, self.max_tile_size)

    class FusedGCN(torch.nn.Module):  # as FusedGCNModule.py:7-18
        def __init__(self, feat_dim, embed_dim, num_classes, adj, num_threads):
            super().__init__()
            schedule = torch.ops.sw_gcn.inspect_vt_ro(adj, feat_dim, embed_dim, 500000, num_threads)
            self.conv1 = FusedGCNLayer(feat_dim, embed_dim, 128, adj, schedule, num_threads)
            self.conv2 = FusedGCNLayer(embed_dim, num_classes, 128, adj, schedule, num_threads)

        def forward(self, x):
            return self.conv2(self.conv1(x).relu())
    return FusedGCN


def test_two_layer_gcn_forward_and_backward(built_lib):
    import torch
    torch.manual_seed(0)
    n, feat, hid, cls = 3000, 100, 64, 47
    g = synth.rmat_gcn(6, n, 12)
    adj = torch.sparse_csr_tensor(torch.from_numpy(g[0]), torch.from_numpy(g[1]), torch.from_numpy(g[2]), size=(n, n)).cuda()
    dense = adj.to_dense().double()
    model = _layers(torch)(feat, hid, cls, adj, 8)
    x = torch.from_numpy(synth.normal(2, (n, feat))).cuda().requires_grad_(True)
    out = model(x)
    w1, w2 = model.conv1.weight.double(), model.conv2.weight.double()
    xd = x.detach().double().requires_grad_(True)
    w1d, w2d = w1.detach().requires_grad_(True), w2.detach().requires_grad_(True)
    want = dense @ ((dense @ (xd @ w1d.t())).relu() @ w2d.t())
    common.assert_close(out.detach().cpu().numpy(), want.detach().cpu().numpy(), "sw_gcn forward")
    loss_w = torch.from_numpy(synth.uniform(9, (n, cls))).cuda()
    (out * loss_w).sum().backward()
    (want * loss_w.double()).sum().backward()
    # the adjacency of a GCN is symmetric, so multiplying the gradient by A (as the reference does) is A^T dY
    common.assert_close(model.conv1.weight.grad.cpu().numpy(), w1d.grad.cpu().numpy(), "dW1")
    common.assert_close(model.conv2.weight.grad.cpu().numpy(), w2d.grad.cpu().numpy(), "dW2")
    common.assert_close(x.grad.cpu().numpy(), xd.grad.cpu().numpy(), "dX")


def test_other_operators(built_lib):
    import torch
    import tile_fusion_b200.sw_gcn  # noqa: F401
    n = 1500
    g = synth.rmat_gcn(4, n, 8)
    adj = torch.sparse_csr_tensor(torch.from_numpy(g[0]), torch.from_numpy(g[1]), torch.from_numpy(g[2]), size=(n, n)).cuda()
    x = torch.from_numpy(synth.normal(2, (n, 32))).cuda()
    w = torch.from_numpy(synth.glorot(3, 48, 32)).cuda()
    want = (adj.to_dense().double() @ (x.double() @ w.double().t())).cpu().numpy()
    sched = torch.ops.sw_gcn.inspect(adj, 128)
    assert len(sched) == 3 and sched[0].dtype == torch.int32 and int(sched[0][2]) >= int(sched[0][1]) > 0
    for got in (torch.ops.sw_gcn.fusedGeMMSpMM(adj, x, w, sched, 4), torch.ops.sw_gcn.unfused_gcn_forward(adj, x, w, 4),
                torch.ops.sw_gcn.geMMSpMM_f_bw(adj, x, w, sched, 4)):
        common.assert_close(got.cpu().numpy(), want, "sw_gcn forward variants")
    af = torch.sparse.mm(adj, x)
    common.assert_close(torch.ops.sw_gcn.cachedSpMMGeMM(af, w, 4).cpu().numpy(), want, "cachedSpMMGeMM")
