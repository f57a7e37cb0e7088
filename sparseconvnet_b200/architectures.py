"""Network builders used by the benchmark configurations: VGG-style, pre-activated ResNet and
U-Net stacks of the inference-path modules.  They produce the same module trees (hence the
same ``state_dict`` keys) as the reference's builders
(sparseconvnet/networkArchitectures.py:9-130 SparseVggNet, :132-200 SparseResNet,
:203-257 UNet)."""
import sparseconvnet_b200 as scn


def _plus_branch(dimension, n_in, planes, depth):
    """A 'Plus' side branch: `depth` stride-2 steps down, then back up, submanifold
    convolutions at every scale on the way."""
    seq = scn.Sequential()
    for level in range(depth):
        seq.add(scn.Convolution(dimension, n_in if level == 0 else planes, planes, 3, 2, False))
        seq.add(scn.BatchNormReLU(planes))
        seq.add(scn.SubmanifoldConvolution(dimension, planes, planes, 3, False))
        seq.add(scn.BatchNormReLU(planes))
    seq.add(scn.Deconvolution(dimension, planes, planes, 3, 2, False))
    for _ in range(depth - 1):
        seq.add(scn.BatchNormReLU(planes))
        seq.add(scn.SubmanifoldConvolution(dimension, planes, planes, 3, False))
        seq.add(scn.BatchNormReLU(planes))
        seq.add(scn.Deconvolution(dimension, planes, planes, 3, 2, False))
    return seq


def SparseVggNet(dimension, nInputPlanes, layers):
    """layers: 'MP' | ['MP', size, stride] | 'C3/2' | ['C3/2', n] | ['C', n] |
    ['C', n, n1[, n2[, n3]]] (the last form adds 'Plus' side branches 1..3 scales down)."""
    n_planes = nInputPlanes
    m = scn.Sequential()
    for x in layers:
        if x == "MP":
            m.add(scn.MaxPooling(dimension, 3, 2))
        elif x[0] == "MP":
            m.add(scn.MaxPooling(dimension, x[1], x[2]))
        elif x == "C3/2":
            m.add(scn.Convolution(dimension, n_planes, n_planes, 3, 2, False))
            m.add(scn.BatchNormReLU(n_planes))
        elif x[0] == "C3/2":
            m.add(scn.Convolution(dimension, n_planes, x[1], 3, 2, False))
            n_planes = x[1]
            m.add(scn.BatchNormReLU(n_planes))
        elif x[0] == "C" and len(x) == 2:
            m.add(scn.SubmanifoldConvolution(dimension, n_planes, x[1], 3, False))
            n_planes = x[1]
            m.add(scn.BatchNormReLU(n_planes))
        elif x[0] == "C" and 3 <= len(x) <= 5:
            table = scn.ConcatTable()
            table.add(scn.SubmanifoldConvolution(dimension, n_planes, x[1], 3, False))
            for depth, planes in enumerate(x[2:], start=1):
                table.add(_plus_branch(dimension, n_planes, planes, depth))
            m.add(table)
            m.add(scn.JoinTable())
            n_planes = sum(x[1:])
            m.add(scn.BatchNormReLU(n_planes))
    return m


def SparseResNet(dimension, nInputPlanes, layers):
    """Pre-activated ResNet; layers = [[block_type, planes, repetitions, stride], ...] with
    block_type 'b...' (basic block)."""
    n_planes = nInputPlanes
    m = scn.Sequential()

    def down(n_in, n_out, stride, index):
        conv = scn.Convolution(dimension, n_in, n_out, 3, stride, False)
        # layers from here on that go down by the same stride: their grids and rulebooks can be built together
        conv.levels_below = sum(1 for layer in layers[index:] if layer[3] == stride)
        return conv

    def shortcut(n_in, n_out, stride, index):
        if stride > 1:
            return down(n_in, n_out, stride, index)
        if n_in != n_out:
            return scn.NetworkInNetwork(n_in, n_out, False)
        return scn.Identity()

    for index, (block_type, n, reps, stride) in enumerate(layers):
        for rep in range(reps):
            if block_type[0] == "b":
                if rep == 0:
                    m.add(scn.BatchNormReLU(n_planes))
                    first = (scn.SubmanifoldConvolution(dimension, n_planes, n, 3, False) if stride == 1
                             else down(n_planes, n, stride, index))
                    main = scn.Sequential().add(first).add(scn.BatchNormReLU(n)).add(
                        scn.SubmanifoldConvolution(dimension, n, n, 3, False))
                    m.add(scn.ConcatTable().add(main).add(shortcut(n_planes, n, stride, index)))
                else:
                    main = scn.Sequential().add(scn.BatchNormReLU(n_planes)).add(
                        scn.SubmanifoldConvolution(dimension, n_planes, n, 3, False)).add(
                        scn.BatchNormReLU(n)).add(scn.SubmanifoldConvolution(dimension, n, n, 3, False))
                    m.add(scn.ConcatTable().add(main).add(scn.Identity()))
            n_planes = n
            m.add(scn.AddTable())
    m.add(scn.BatchNormReLU(n_planes))
    return m


def UNet(dimension, reps, nPlanes, residual_blocks=False, downsample=[2, 2], leakiness=0,
         n_input_planes=-1):
    """U-Net of submanifold convolutions: `reps` blocks per level, a strided Convolution down and
    the matching Deconvolution up, skip connection joined by concatenation."""

    def block(m, a, b):
        if residual_blocks:
            m.add(scn.ConcatTable()
                  .add(scn.Identity() if a == b else scn.NetworkInNetwork(a, b, False))
                  .add(scn.Sequential()
                       .add(scn.BatchNormLeakyReLU(a, leakiness=leakiness))
                       .add(scn.SubmanifoldConvolution(dimension, a, b, 3, False))
                       .add(scn.BatchNormLeakyReLU(b, leakiness=leakiness))
                       .add(scn.SubmanifoldConvolution(dimension, b, b, 3, False))))
            m.add(scn.AddTable())
        else:
            m.add(scn.Sequential()
                  .add(scn.BatchNormLeakyReLU(a, leakiness=leakiness))
                  .add(scn.SubmanifoldConvolution(dimension, a, b, 3, False)))

    def down(planes):
        conv = scn.Convolution(dimension, planes[0], planes[1], downsample[0], downsample[1], False)
        conv.levels_below = len(planes) - 1  # the encoder goes this many levels further down
        return conv

    def level(planes, n_in=-1):
        m = scn.Sequential()
        for _ in range(reps):
            block(m, n_in if n_in != -1 else planes[0], planes[0])
            n_in = -1
        if len(planes) > 1:
            down_up = (scn.Sequential()
                       .add(scn.BatchNormLeakyReLU(planes[0], leakiness=leakiness))
                       .add(down(planes))
                       .add(level(planes[1:]))
                       .add(scn.BatchNormLeakyReLU(planes[1], leakiness=leakiness))
                       .add(scn.Deconvolution(dimension, planes[1], planes[0], downsample[0], downsample[1], False)))
            m.add(scn.ConcatTable().add(scn.Identity()).add(down_up))
            m.add(scn.JoinTable())
            for i in range(reps):
                block(m, planes[0] * (2 if i == 0 else 1), planes[0])
        return m

    return level(nPlanes, n_input_planes)


def FullyConvolutionalNet(dimension, reps, nPlanes, residual_blocks=False, downsample=[2, 2]):
    """Fully-convolutional network for per-voxel prediction (reference:
    networkArchitectures.py:259-312): `reps` blocks per level, a strided Convolution down, the
    deeper levels, then UnPooling back to this level's sites; the coarse result is concatenated to
    the level's own features, so the output has sum(nPlanes) planes at the input's sites."""

    def block(m, a, b):
        if residual_blocks:
            shortcut = scn.Identity() if a == b else scn.NetworkInNetwork(a, b, False)
            body = (scn.Sequential()
                    .add(scn.BatchNormReLU(a)).add(scn.SubmanifoldConvolution(dimension, a, b, 3, False))
                    .add(scn.BatchNormReLU(b)).add(scn.SubmanifoldConvolution(dimension, b, b, 3, False)))
            m.add(scn.ConcatTable().add(shortcut).add(body)).add(scn.AddTable())
        else:
            m.add(scn.Sequential().add(scn.BatchNormReLU(a))
                  .add(scn.SubmanifoldConvolution(dimension, a, b, 3, False)))

    def down(planes):
        conv = scn.Convolution(dimension, planes[0], planes[1], downsample[0], downsample[1], False)
        conv.levels_below = len(planes) - 1
        return conv

    def level(planes):
        m = scn.Sequential()
        for _ in range(reps):
            block(m, planes[0], planes[0])
        if len(planes) > 1:
            deeper = (scn.Sequential()
                      .add(scn.BatchNormReLU(planes[0]))
                      .add(down(planes))
                      .add(level(planes[1:]))
                      .add(scn.UnPooling(dimension, downsample[0], downsample[1])))
            m.add(scn.ConcatTable().add(scn.Identity()).add(deeper))
            m.add(scn.JoinTable())
        return m

    return level(nPlanes)
