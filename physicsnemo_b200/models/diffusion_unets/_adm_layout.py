"""Layout of the ADM ("Dhariwal") U-Net shared by ``DhariwalUNet`` and ``TopoDiff``: which modules sit under which
ModuleDict key, in execution order, and how wide they are.  The keys (``"{side}x{side}_conv|_down|_block{i}|_in0|_in1|_up"``)
are the checkpoint contract of ``physicsnemo/models/diffusion_unets/dhariwal_unet.py``."""
from dataclasses import dataclass


@dataclass(frozen=True)
class Stage:
    """One entry of the U-Net layout: ModuleDict key, ``"conv"`` or ``"block"``, channel widths, block options."""

    key: str
    kind: str
    width_in: int
    width_out: int
    options: tuple = ()


def unet_layout(resolution: int, first_in: int, base_width: int, multipliers, blocks_per_level: int, attention_sides):
    """Encoder and decoder stages of the EDM-style U-Net, in execution order.

    Encoder, level by level: an input convolution (finest level) or a down-sampling block, then ``blocks_per_level``
    residual blocks.  Decoder, coarsest level first: two bottleneck blocks (the first with attention) or an up-sampling
    block, then ``blocks_per_level + 1`` blocks that each consume one encoder output as skip connection.
    """
    encoder, width = [], first_in
    for depth, mult in enumerate(multipliers):
        side = resolution // 2 ** depth
        tag, target = f"{side}x{side}", base_width * mult
        if depth:
            encoder.append(Stage(f"{tag}_down", "block", width, width, (("down", True),)))
        else:
            encoder.append(Stage(f"{tag}_conv", "conv", width, target))
            width = target
        for b in range(blocks_per_level):
            encoder.append(Stage(f"{tag}_block{b}", "block", width, target, (("attention", side in attention_sides),)))
            width = target
    pending_skips = [stage.width_out for stage in encoder]
    decoder, coarsest = [], len(multipliers) - 1
    for depth in range(coarsest, -1, -1):
        side = resolution // 2 ** depth
        tag, target = f"{side}x{side}", base_width * multipliers[depth]
        if depth == coarsest:
            decoder.append(Stage(f"{tag}_in0", "block", width, width, (("attention", True),)))
            decoder.append(Stage(f"{tag}_in1", "block", width, width))
        else:
            decoder.append(Stage(f"{tag}_up", "block", width, width, (("up", True),)))
        for b in range(blocks_per_level + 1):
            decoder.append(Stage(f"{tag}_block{b}", "block", width + pending_skips.pop(), target,
                                  (("attention", side in attention_sides),)))
            width = target
    return encoder, decoder, width
