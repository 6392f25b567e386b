"""ACT controller: traces a model, decides bits / group size / padding per layer and
swaps the supported modules for their compressed-activation versions.

Public surface of Activation_Compression/controller.py:18-390: `Controller(model,
config, train_loader, criterion, test)`, `.iterate()`, `.warp_model(graph_mode,
quantizer)`, `.traced_model`, `.meta`, `.target_dict`, and the helpers
`find_group_size`, `assign_tensor_meta`, `compute_activation_size_in_bytes`.
Config keys are the reference's: default_bits, auto_precision, DIVISION,
AVG_ALAM, AVG_ALAM_BTS, group_size, batch_size, fp8, analyze, depth_point_conv,
rms_norm.  Differences: shapes are propagated on the meta device (no GPU needed
to build the plan); the low-frequency-energy probe that picks DIVISION layers is
a research analysis outside this path, so DIVISION applies to no layer unless
`division_targets` lists them; `min_activation_mib` (default 10, the reference's
constant) sets the size below which a layer is left alone.
"""
from __future__ import annotations

import copy

import torch
import torch.fx as FX
from torch import nn
from torch.fx.passes.shape_prop import ShapeProp

from .layers import DOConv1d, DOConv2d, DOConv3d, DODepthPointConv2d, DOLinear, RMSNorm
from .modules.activations.act_layers import DOGELU, DOMaxPool2d, DOReLU_Variance, DOSiLU
from .modules.normalization.normalization_layers import DOBatchNorm2d, DOLayerNorm, DOSyncBatchNorm2d
from .quantizer import Quantizer

_SUPPORTED = (nn.Linear, nn.Conv1d, nn.Conv2d, nn.Conv3d, nn.BatchNorm2d, nn.SyncBatchNorm,
              nn.ReLU, nn.ReLU6, nn.SiLU, nn.GELU)
# not in the reference's swap list (controller.py:87); on unless the config says
# compress_layernorm=False
_EXTENSIONS = (nn.LayerNorm,)


def assign_tensor_meta(node):
    """tensor_meta of the first tensor argument of a node (controller.py:355-361)."""
    for arg in node.args:
        if isinstance(arg, torch.fx.Node) and arg.op != "get_attr":
            tm = arg.meta.get("tensor_meta", None)
            if tm is not None:
                return tm
    return None


def find_group_size(S, bits, max_group=512, special=False):
    """Largest of 512/256/128/64 (1024 too when `special`) dividing S; else 256 with
    zero padding (controller.py:364-378)."""
    groups = [1024, 512, 256, 128, 64] if special else [512, 256, 128, 64]
    if bits in (1, 2, 4, 8):
        for gs in groups:
            if S % gs == 0:
                return gs, False
    return 256, True


def compute_activation_size_in_bytes(node):
    """Size in MiB of the node's output (controller.py:381-390; the name says bytes)."""
    tm = node.meta.get("tensor_meta", None)
    if tm is None:
        return 0
    numel = 1
    for s in tm.shape:
        numel *= s
    return numel * torch.tensor([], dtype=tm.dtype).element_size() / (1024 ** 2)


class Controller:
    def __init__(self, model, config, train_loader=None, criterion=None, test=True, input_shape=None,
                 device=None):
        self.device = device if device is not None else ("cuda" if torch.cuda.is_available() else "cpu")
        self.model = model.to(self.device)
        self.config = config
        self.train_loader = train_loader
        self.criterion = criterion
        if input_shape is None:
            x, _ = next(iter(self.train_loader))
            input_shape = x.shape[1:]
        self.input_shape = tuple(input_shape)
        self.quantizer = Quantizer(config, {})
        self.quantizer.filter_tensors(self.model.named_parameters())
        self.meta = {"group_size": config.get("group_size", 256), "fp8": config.get("fp8", False),
                     "analyze": config.get("analyze", False)}
        self.layer_clamp = 3.0
        self.traced_model = None
        self.target_dict = {}
        self.fused_bn_relu = []
        if not test:
            self.warp_model(quantizer=True)

    def iterate(self, criterion=None, trainloader=None):
        self.quantizer.iterate(self.model, criterion or self.criterion, trainloader or self.train_loader)

    # ------------------------------------------------------------------ planning
    def _plan(self, traced):
        named = dict(traced.named_modules())
        # shapes are propagated through a bf16 copy on the meta device (what autocast
        # training sees), leaving the real parameters where they are
        meta_model = copy.deepcopy(traced).to(device="meta", dtype=torch.bfloat16)
        fake = torch.empty(self.config["batch_size"], *self.input_shape, dtype=torch.bfloat16, device="meta")
        ShapeProp(meta_model).propagate(fake)
        threshold = self.config.get("min_activation_mib", 10)
        pairs = {}
        for node in meta_model.graph.nodes:
            if node.op != "call_module":
                continue
            mod = named[node.target]
            if not isinstance(mod, _SUPPORTED) and not (
                    isinstance(mod, _EXTENSIONS) and self.config.get("compress_layernorm", True)
                    and not self.config.get("rms_norm", False)):
                continue
            if compute_activation_size_in_bytes(node) <= threshold:
                continue
            tm = assign_tensor_meta(node)
            if tm is None:
                continue
            pairs[node.target] = {"mod": mod, "tensor_meta": tm}
        return pairs

    def _layer_meta(self, target, mod, tm):
        bits = self.quantizer.bits[target]
        entry = {"tensor_meta": tm, "pack_only": False, "bits": bits}
        if isinstance(mod, (nn.ReLU, nn.ReLU6)):
            entry["pack_only"], entry["bits"] = True, 1
        shape = tuple(tm.shape)
        is_bn = isinstance(mod, (nn.BatchNorm2d, nn.SyncBatchNorm))
        if len(shape) >= 3 and is_bn:
            per = shape[0]
            for d in shape[2:]:
                per *= d
            N = shape[1]
        else:
            per = 1
            for d in shape[1:]:
                per *= d
            N = shape[0]
        group_size, act_padding = find_group_size(per, bits, special=is_bn)
        if is_bn:
            # this backend groups the normalised tensor sample-major like every other
            # layer, so the group size must divide a sample, not a channel
            per_sample = 1
            for d in shape[1:]:
                per_sample *= d
            group_size, act_padding = find_group_size(per_sample, bits, special=True)
            N = shape[0]
            per = per_sample
        G = (per + group_size - 1) // group_size
        entry.update({"group_size": group_size, "act_padding": act_padding, "N": N, "NG": N * G})
        if self.config.get("AVG_ALAM", None) is not None and not isinstance(
                mod, (nn.Linear, nn.Conv1d, nn.Conv2d, nn.Conv3d)):
            entry.update({"AVG_ALAM": self.config["AVG_ALAM"], "ALAM_BITS": self.config["AVG_ALAM_BTS"]})
        else:
            entry.update({"AVG_ALAM": False, "ALAM_BITS": 0})
        division = self.config.get("DIVISION", None)
        entry["DIVISION"] = division if (division is not None and target in self.config.get("division_targets", ())) else None
        return entry

    def _replacement(self, target, mod):
        kw = dict(target_name=target, meta=self.meta)
        if isinstance(mod, nn.Linear):
            new = DOLinear(mod.in_features, mod.out_features, clamp_alpha=self.layer_clamp, **kw)
            if mod.bias is None:
                new.bias = None
        elif isinstance(mod, nn.Conv1d):
            new = DOConv1d(mod.in_channels, mod.out_channels, mod.kernel_size, mod.stride, mod.padding,
                           mod.dilation, mod.groups, mod.padding_mode, clamp_alpha=self.layer_clamp,
                           bias=mod.bias is not None, **kw)
        elif isinstance(mod, nn.Conv2d):
            if self.config.get("depth_point_conv", False):
                return DODepthPointConv2d(mod.in_channels, mod.out_channels, mod.kernel_size, mod.stride,
                                          mod.padding, mod.dilation, mod.groups, mod.padding_mode,
                                          acc_var=self.layer_clamp, **kw)
            new = DOConv2d(mod.in_channels, mod.out_channels, mod.kernel_size, mod.stride, mod.padding,
                           mod.dilation, mod.groups, mod.padding_mode, clamp_alpha=self.layer_clamp,
                           bias=mod.bias is not None, **kw)
        elif isinstance(mod, nn.Conv3d):
            new = DOConv3d(mod.in_channels, mod.out_channels, mod.kernel_size, mod.stride, mod.padding,
                           mod.dilation, mod.groups, mod.padding_mode, clamp_alpha=self.layer_clamp,
                           bias=mod.bias is not None, **kw)
        elif isinstance(mod, nn.SyncBatchNorm):
            new = DOSyncBatchNorm2d(mod.num_features, mod.eps, mod.momentum, mod.affine,
                                    mod.track_running_stats, mod.process_group, **kw)
        elif isinstance(mod, nn.BatchNorm2d):
            new = DOBatchNorm2d(mod.num_features, mod.eps, mod.momentum, mod.affine,
                                mod.track_running_stats, **kw)
        elif isinstance(mod, nn.LayerNorm):
            new = DOLayerNorm(mod.normalized_shape, mod.eps, mod.elementwise_affine, mod.bias is not None, **kw)
        elif isinstance(mod, nn.ReLU6):
            return DOReLU_Variance(inplace=False, relu=False, relu6=True, **kw)
        elif isinstance(mod, nn.ReLU):
            return DOReLU_Variance(inplace=False, relu=True, relu6=False, **kw)
        elif isinstance(mod, nn.SiLU):
            return DOSiLU(inplace=False, **kw)
        elif isinstance(mod, nn.GELU):
            return DOGELU(inplace=False, approximate=mod.approximate, **kw)
        else:
            raise TypeError(type(mod))
        with torch.no_grad():
            for name in ("weight", "bias", "running_mean", "running_var", "num_batches_tracked"):
                src, dst = getattr(mod, name, None), getattr(new, name, None)
                if src is not None and dst is not None:
                    dst.copy_(src)
        return new

    @staticmethod
    def _fuse_bn_relu(traced):
        """BatchNorm whose only consumer is a plain ReLU: the BatchNorm module takes the ReLU
        over (one forward kernel, no ReLU backward pass; the reference's norm+activation fusion,
        triton_kernel/norm_act_fusion/bn_act_fusion.py) and the ReLU node leaves the graph.
        Returns the fused BatchNorm targets."""
        fused = []
        for node in list(traced.graph.nodes):
            if node.op != "call_module" or len(node.users) != 1:
                continue
            bn = traced.get_submodule(node.target)
            if type(bn) is not DOBatchNorm2d:
                continue
            user = next(iter(node.users))
            if user.op != "call_module" or len(user.args) != 1 or user.args[0] is not node:
                continue
            relu = traced.get_submodule(user.target)
            if not (isinstance(relu, DOReLU_Variance) and relu.relu and not relu.relu6):
                continue
            bn.fuse_relu = True
            user.replace_all_uses_with(node)
            traced.graph.erase_node(user)
            fused.append(node.target)
        return fused

    @staticmethod
    def _fuse_bn_add_relu(traced):
        """relu(batch_norm(x) + skip), the end of a residual block (Model/CNN/ResNetV1.py:48-49 of
        the reference): the BatchNorm module takes the add and the ReLU over.  The pattern is a
        BatchNorm whose only consumer is an add whose only consumer is a plain ReLU; the BatchNorm
        call moves to the add's place (the skip operand may be computed after it) with the skip
        as its second argument.  Returns the fused BatchNorm targets."""
        import operator
        adds = (operator.add, operator.iadd, torch.add)
        fused = []
        for node in list(traced.graph.nodes):
            if node.op != "call_module" or len(node.users) != 1 or len(node.args) != 1:
                continue
            bn = traced.get_submodule(node.target)
            if type(bn) is not DOBatchNorm2d or bn.fuse_relu:
                continue
            add = next(iter(node.users))
            if (add.op != "call_function" or add.target not in adds or len(add.args) != 2 or add.kwargs
                    or len(add.users) != 1):
                continue
            other = add.args[1] if add.args[0] is node else add.args[0]
            if other is node or not isinstance(other, FX.Node):
                continue
            user = next(iter(add.users))
            if user.op != "call_module" or len(user.args) != 1:
                continue
            relu = traced.get_submodule(user.target)
            if not (isinstance(relu, DOReLU_Variance) and relu.relu and not relu.relu6):
                continue
            with traced.graph.inserting_before(add):
                new = traced.graph.call_module(node.target, args=(node.args[0], other))
            bn.fuse_relu = True
            user.replace_all_uses_with(new)
            traced.graph.erase_node(user)
            traced.graph.erase_node(add)
            traced.graph.erase_node(node)
            fused.append(new.target)
        return fused

    @staticmethod
    def _fuse_add_layer_norm(traced):
        """s = a + b; y = layer_norm(s), the pre-norm transformer block (Model/ViT/ViT.py:84-86 of
        the reference), where s also feeds the next residual addition: the LayerNorm module takes
        the addition over and returns (y, s).  Its forward kernel then forms s from a and b while it
        reads them (the separate addition and the re-read of its result fall away), and its backward
        kernel adds the gradient that reaches s from its other consumers to the LayerNorm's own
        input gradient, which autograd would do with one more pass.  Operands of different shapes
        or types are added by the module the ordinary way.  Returns the fused targets."""
        import operator
        fused = []
        for node in list(traced.graph.nodes):
            if node.op != "call_module" or len(node.args) != 1 or node.kwargs:
                continue
            if type(traced.get_submodule(node.target)) is not DOLayerNorm:
                continue
            add = node.args[0]
            if (not isinstance(add, FX.Node) or add.op != "call_function" or add.target not in (operator.add, torch.add)
                    or len(add.args) != 2 or add.kwargs):
                continue
            a, b = add.args
            if not (isinstance(a, FX.Node) and isinstance(b, FX.Node)):
                continue
            # at the addition's place: its other consumers may come before the LayerNorm call
            with traced.graph.inserting_after(add):
                new = traced.graph.call_module(node.target, args=(a, b))
            with traced.graph.inserting_after(new):
                total = traced.graph.call_function(operator.getitem, (new, 1))
            with traced.graph.inserting_after(new):
                y = traced.graph.call_function(operator.getitem, (new, 0))
            node.replace_all_uses_with(y)
            traced.graph.erase_node(node)
            add.replace_all_uses_with(total)
            traced.graph.erase_node(add)
            fused.append(new.target)
        return fused

    @staticmethod
    def _fork_block_outputs(traced, targets):
        """A block output relu(batch_norm(x) + skip) usually feeds two consumers, the next block's
        first convolution and its skip (or its downsample convolution).  Autograd would add their
        two gradients with a kernel of its own; instead the fused BatchNorm returns its output
        twice, one value per consumer, and its backward adds the two gradients inside the mask
        pass it runs anyway.  Applied where the fused node has exactly two users."""
        import operator
        forked = []
        for node in list(traced.graph.nodes):
            if node.op != "call_module" or node.target not in targets or len(node.users) != 2:
                continue
            bn = traced.get_submodule(node.target)
            if type(bn) is not DOBatchNorm2d or not bn.fuse_relu or len(node.args) != 2:
                continue
            users = list(node.users)
            with traced.graph.inserting_after(node):
                second = traced.graph.call_function(operator.getitem, (node, 1))
            with traced.graph.inserting_after(node):
                first = traced.graph.call_function(operator.getitem, (node, 0))
            users[0].replace_input_with(node, first)
            users[1].replace_input_with(node, second)
            bn.fork = True
            forked.append(node.target)
        return forked

    # ------------------------------------------------------------------ rewrite
    def warp_model(self, graph_mode=False, quantizer=False):
        traced = FX.symbolic_trace(self.model)
        pairs = self._plan(traced)
        self.target_dict = pairs
        if quantizer:
            self.quantizer.bits = {t: self.config["default_bits"] for t in pairs}
            self.iterate()
            self.meta["batch_size"] = self.config["batch_size"]
            for target, d in pairs.items():
                self.meta[f"{target}"] = self._layer_meta(target, d["mod"], d["tensor_meta"])
            for target, d in pairs.items():
                new_mod = self._replacement(target, d["mod"])
                parent_path, _, child = target.rpartition(".")
                setattr(traced.get_submodule(parent_path), child, new_mod)
            if self.config.get("rms_norm", False):
                for name, mod in list(traced.named_modules()):
                    if isinstance(mod, nn.LayerNorm):
                        parent_path, _, child = name.rpartition(".")
                        setattr(traced.get_submodule(parent_path), child, RMSNorm(mod.normalized_shape[-1]))
            if self.config.get("compress_maxpool", True):
                # not in the reference's swap list (controller.py:87): max-pool layers keep a 4-bit
                # argmax for backward when their input is channels-last
                for name, mod in list(traced.named_modules()):
                    if type(mod) is nn.MaxPool2d:
                        parent_path, _, child = name.rpartition(".")
                        setattr(traced.get_submodule(parent_path), child,
                                DOMaxPool2d(mod.kernel_size, mod.stride, mod.padding, mod.dilation,
                                            mod.return_indices, mod.ceil_mode))
            self.fused_add_layer_norm = []
            if self.config.get("fuse_add_layer_norm", True):
                self.fused_add_layer_norm = self._fuse_add_layer_norm(traced)
            self.fused_bn_add_relu = []
            if self.config.get("fuse_bn_relu", True):
                if self.config.get("fuse_bn_add_relu", True):
                    self.fused_bn_add_relu = self._fuse_bn_add_relu(traced)
                    self.forked_block_outputs = []
                    if self.config.get("fork_block_outputs", True):
                        self.forked_block_outputs = self._fork_block_outputs(traced, set(self.fused_bn_add_relu))
                self.fused_bn_relu = self._fuse_bn_relu(traced)
            traced.graph.eliminate_dead_code()
            traced.graph.lint()
            traced.recompile()
        if "fused_dw" in self.config:
            from .modules import ops as _ops
            _ops.set_fused_dw(self.config["fused_dw"])
        if graph_mode:
            torch.backends.cuda.matmul.allow_tf32 = True
            torch.backends.cudnn.allow_tf32 = True
            torch.set_float32_matmul_precision("high")
        self.traced_model = traced.to(self.device).train()
        return self.traced_model
