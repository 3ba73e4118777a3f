"""Complete a prompt with a trained checkpoint:

    python examples/inference_example/generate.py <checkpoint dir> "Once upon a time" --max-tokens 32

The checkpoint directory holds the per-layer weight files, ``config.yml`` and ``vocab.json``.
"""

import argparse
from pathlib import Path

from scaling_b200.transformer.inference import TransformerInferenceModule, sample_argmax, sample_temperature

if __name__ == "__main__":
    parser = argparse.ArgumentParser()
    parser.add_argument("checkpoint", type=Path)
    parser.add_argument("prompt", type=str)
    parser.add_argument("--max-tokens", type=int, default=32)
    parser.add_argument("--temperature", type=float, default=0.0)
    parser.add_argument("--devices", type=int, nargs="+", default=[0])
    args = parser.parse_args()
    model = TransformerInferenceModule.from_checkpoint(args.checkpoint, devices=args.devices, use_flash_attention=True)
    sample = sample_argmax if args.temperature == 0.0 else (lambda logits: sample_temperature(logits, args.temperature))
    out = model.generate(max_tokens=args.max_tokens, input_text=args.prompt, sample_fn=sample)
    print(out.completion_text)
