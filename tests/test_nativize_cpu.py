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
