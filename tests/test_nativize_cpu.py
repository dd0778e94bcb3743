"""Planning done by layers.nativize on a residual network (no kernels run: CPU only)."""
import torch

from pipedream_b200 import layers, stages


def test_resnet_plan_keeps_names_and_fuses_tails():
    torch.manual_seed(0)
    st = stages.resnet50(1).stages()[0]
    keys = list(st.state_dict().keys())
    params = [n for n, _ in st.named_parameters()]
    nat = layers.nativize(st)
    assert list(nat.state_dict().keys()) == keys
    assert [n for n, _ in nat.named_parameters()] == params
    assert sum(p.numel() for p in nat.parameters()) == 25557032
    blk = nat.parts[1]          # first bottleneck block: projection shortcut
    assert isinstance(blk, torch.fx.GraphModule)
    assert isinstance(blk.bn1, layers.NativeBatchNorm2d) and blk.bn1.fuse_relu and not blk.bn1.out_nchw
    assert isinstance(blk.conv2, layers.NativeConv2d) and isinstance(blk.conv1, layers.NativeConvGeneric)
    assert blk.bn3.fuse_relu and not blk.bn3.out_nchw          # add + ReLU folded in, result stays padded
    assert isinstance(blk.pd_fork0, layers.NativeFork)
    targets = [n.target for n in blk.graph.nodes if n.op == "call_module"]
    assert targets[-1] == "bn3" and "relu3" not in targets
    assert not nat.parts[0].pool.out_nchw                       # stem -> first block stays padded
    assert nat.parts[16].bn3.out_nchw is False and nat.parts[17]._pd_accepts_padded


def test_stage_boundary_emits_plain_tensors():
    torch.manual_seed(0)
    sts = [layers.nativize(s) for s in stages.resnet50(6).stages()]
    for st in sts[:-1]:
        last = st.parts[len(st.parts) - 1]
        assert last.bn3.out_nchw            # what crosses a stage boundary is a contiguous NCHW tensor


def test_vgg_and_gnmt_stages_keep_their_own_forward():
    v = stages.vgg16("gpus=1").stages()[0]
    assert layers.nativize(v) is v


def test_balanced_cuts_are_optimal():
    import itertools
    import random
    rnd = random.Random(7)
    for _ in range(30):
        n = rnd.randint(3, 9)
        k = rnd.randint(1, n)
        costs = [rnd.randint(1, 50) for _ in range(n)]
        sizes = stages._balanced_cuts(costs, k)
        assert len(sizes) == k and sum(sizes) == n and min(sizes) >= 1
        got, i = 0, 0
        for sz in sizes:
            got = max(got, sum(costs[i:i + sz]))
            i += sz
        best = min(max(sum(costs[a:b]) for a, b in zip((0,) + cut, cut + (n,)))
                   for cut in itertools.combinations(range(1, n), k - 1))
        assert got == best


def test_resnet_partitions_cover_the_network_and_report_their_boundaries():
    for k in (1, 3, 8):
        pkg = stages.resnet50(k)
        sts = pkg.stages()
        assert len(sts) == k and sum(len(s.parts) for s in sts) == 18
        assert sum(p.numel() for s in sts for p in s.parameters()) == 25557032
        shapes = pkg.boundary_shapes(2)
        x = torch.randn(*shapes["input0"])
        with torch.no_grad():
            for i, s in enumerate(sts):
                s.eval()
                x = s(x)
                assert tuple(x.shape) == tuple(shapes["out%d" % i])
        assert abs(2 * sum(pkg.stage_macs()) / 1e9 - 8.18) < 0.01       # forward GFLOP per sample
