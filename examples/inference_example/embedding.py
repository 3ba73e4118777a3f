"""Sentence embeddings from a checkpoint trained with the embedding head and the contrastive loss:

    python examples/inference_example/embedding.py <checkpoint dir> "first sentence" "second sentence"
"""

import argparse
from pathlib import Path

import torch

from scaling_b200.transformer.inference import TransformerInferenceModule

if __name__ == "__main__":
    parser = argparse.ArgumentParser()
    parser.add_argument("checkpoint", type=Path)
    parser.add_argument("sentences", type=str, nargs="+")
    parser.add_argument("--instruction", type=str, default="")
    args = parser.parse_args()
    model = TransformerInferenceModule.from_checkpoint(args.checkpoint, devices=[0])
    emb = model.encode(args.sentences, instruction=args.instruction, convert_to_tensor=True)
    emb = torch.nn.functional.normalize(emb.float(), dim=-1)
    print("embeddings:", tuple(emb.shape))
    print("cosine similarities:\n", emb @ emb.T)
