"""Datasets, blending, tokenizer and sampling helpers (CPU)."""

import json
from pathlib import Path

import numpy as np
import pytest
import torch

from scaling_b200.core.data import BlendedDatasetConfig, MemoryMapDatasetBuilder
from scaling_b200.core.data.blended_dataset import (build_blend_index, weights_by_num_docs,
                                                    weights_examples_proportional)
from scaling_b200.transformer.data import (EmbeddingDataset, FinetuningChatDataset, FinetuningTextBlendedDataset,
                                           FinetuningTextDataset, TextBlendedDataset, TextDataset)
from scaling_b200.transformer.inference import sample_argmax, sample_temperature, top_k_transform, top_p_transform
from scaling_b200.transformer.tokenizer import Tokenizer, load_tokenizers

WORDS = ["the", "cat", "sat", "on", "mat", "a", "dog", "ran", "far", "query", "doc", "good", "bad", "find", ":"]


@pytest.fixture()
def tok() -> Tokenizer:
    return Tokenizer.from_words(WORDS)


def _oracle(targets, until_all):
    """The dataset furthest behind its target comes next; stop at the first finished dataset, or let finished ones
    drop out and go on until all are done."""
    t = np.array(targets)
    s = np.zeros(len(t), dtype=np.int64)
    out = []
    while (s < t).any() if until_all else (s < t).all():
        share = np.where(s < t, s / t, np.inf)
        i = int(share.argmin())
        out.append((i, int(s[i])))
        s[i] += 1
    return out


@pytest.mark.parametrize("until_all", [True, False])
@pytest.mark.parametrize("targets", [[5, 3, 9], [1, 1], [7], [100, 1, 33, 33], [2, 4, 8, 16, 32], [12, 12, 12]])
def test_blend_index_matches_greedy_oracle(tmp_path: Path, targets, until_all):
    n = build_blend_index(targets, str(tmp_path / "idx"), until_all=until_all)
    pairs = np.fromfile(tmp_path / "idx.bin", dtype=np.int64).reshape(-1, 2)
    assert n == len(pairs)
    assert [tuple(p) for p in pairs.tolist()] == _oracle(targets, until_all)
    if until_all:
        assert n == sum(targets)  # every dataset gives all it was asked for
    meta = json.loads((tmp_path / "idx.meta.json").read_text())
    assert meta == {"dtype": "int64", "shape": [n, 2]}


def test_blend_weights():
    w = weights_by_num_docs([100, 10], alpha=1.0)
    assert np.allclose(w, [0.5, 0.5])  # alpha 1 keeps the natural proportions: equal multipliers
    w0 = weights_by_num_docs([100, 10], alpha=0.0)
    assert w0[1] / w0[0] == pytest.approx(10.0)  # alpha 0: equal sampling -> the small set is boosted 10x
    e = weights_examples_proportional([100, 10], temperature=1.0, maximum=None)
    assert np.allclose(e, [0.5, 0.5])
    capped = weights_examples_proportional([100, 10], temperature=1.0, maximum=10)
    assert capped[1] / capped[0] == pytest.approx(10.0)
    with pytest.raises(AssertionError):
        weights_examples_proportional([1, 2], temperature=0)


def _text_map(prefix: Path, n_docs: int, seed: int) -> None:
    rng = np.random.default_rng(seed)
    with MemoryMapDatasetBuilder(prefix_path=prefix) as b:
        for _ in range(n_docs):
            b.add(np_array=np.concatenate([rng.integers(1, 50, size=rng.integers(3, 20)), [0]]).astype(np.int32))


def test_text_blended_dataset(tmp_path: Path):
    _text_map(tmp_path / "a", 60, 1)
    _text_map(tmp_path / "b", 15, 2)
    sets = [TextDataset(data_prefix=tmp_path / n, sequence_length=16, seed=3) for n in ("a", "b")]
    cfg = BlendedDatasetConfig(weight_by_num_documents=True, weighted_sampler_alpha=0.5, cache_directory=tmp_path / "cache")
    blend = TextBlendedDataset(seed=3, config=cfg, datasets=sets)
    assert len(blend) > 0
    counts = np.bincount(np.asarray(blend.dataset_indices)[:, 0], minlength=2)
    assert counts[0] > 0 and counts[1] > 0
    item = blend[0]
    batch = blend.collate([blend[i] for i in range(4)])
    assert batch.token_ids.shape == (4, 17)
    assert torch.equal(item.token_ids, sets[int(blend.dataset_indices[0][0])][int(blend.dataset_indices[0][1])].token_ids)
    # a second instance finds the cached index
    again = TextBlendedDataset(seed=3, config=cfg, datasets=sets)
    assert np.array_equal(np.asarray(again.dataset_indices), np.asarray(blend.dataset_indices))
    single = TextBlendedDataset(seed=3, config=cfg, datasets=sets[:1])
    assert len(single) == len(sets[0])


def test_finetuning_text_dataset_json_and_memory_map(tmp_path: Path, tok: Tokenizer):
    records = [{"prompt": "the cat sat", "completion": "on the mat"}, {"prompt": "a dog", "completion": "ran far"}]
    (tmp_path / "ft.json").write_text(json.dumps(records))
    ds = FinetuningTextDataset(tmp_path / "ft.json", sequence_length=12, seed=1, softprompt_n_tokens=2, tokenizer=tok,
                               tokenizer_no_prefix_space=tok, shuffle=False)
    item = ds[0]
    p, c = tok.encode("the cat sat"), tok.encode("on the mat")
    assert item.input_token_ids.tolist()[:2 + len(p) + len(c)] == [0, 0] + p + c
    # loss on the completion and on exactly one end-of-text token
    n_prompt = 2 + len(p)
    assert item.loss_weights.tolist() == [0.0] * (n_prompt - 1) + [1.0] * (len(c) + 1) + [0.0] * (12 - n_prompt - len(c))
    assert item.target_token_ids[n_prompt + len(c) - 1].item() == tok.eos_token_id
    batch = ds.collate([ds[0], ds[1]])
    assert batch.input_token_ids.shape == (2, 12) and batch.input_images is None
    assert FinetuningTextDataset.sync_batch_to_model_parallel(None, batch) is batch

    (tmp_path / "ft.jsonl").write_text("\n".join(json.dumps(r) for r in records) + "\n")
    FinetuningTextDataset.convert_jsonl(tmp_path / "ft.jsonl", tok, tok, tmp_path / "ftmap")
    mm = FinetuningTextDataset(tmp_path / "ftmap", sequence_length=12, seed=1, softprompt_n_tokens=2, tokenizer=tok,
                               tokenizer_no_prefix_space=tok, memory_map_dataset=True, shuffle=False)
    assert torch.equal(mm[0].input_token_ids, item.input_token_ids)
    assert torch.equal(mm[0].loss_weights, item.loss_weights)
    cfg = BlendedDatasetConfig(cache_directory=tmp_path / "c")
    assert len(FinetuningTextBlendedDataset(seed=1, config=cfg, datasets=[ds])) == 2


def test_finetuning_chat_dataset(tmp_path: Path, tok: Tokenizer):
    conv = [{"type": "text", "content": "the cat", "has_loss": False}, {"type": "text", "content": "sat on", "has_loss": True},
            {"type": "text", "content": "a mat", "has_loss": False}]
    (tmp_path / "chat.jsonl").write_text(json.dumps(conv) + "\n")
    ds = FinetuningChatDataset(tmp_path / "chat.jsonl", sequence_length=8, seed=1, softprompt_n_tokens=0, tokenizer=tok,
                               tokenizer_no_prefix_space=tok)
    item = ds[0]
    ids = tok.encode("the cat") + tok.encode("sat on") + tok.encode("a mat")
    assert item.input_token_ids.tolist() == ids[:-1] + [tok.padding_token_id] * (8 - len(ids) + 1)
    assert item.target_token_ids.tolist()[:len(ids) - 1] == ids[1:]
    assert item.loss_weights.tolist() == [0, 1, 1, 0, 0, 0, 0, 0]  # targets "sat", "on" carry the loss
    with pytest.raises(NotImplementedError):
        (tmp_path / "bad.jsonl").write_text(json.dumps([{"type": "audio", "content": "x"}]) + "\n")
        FinetuningChatDataset(tmp_path / "bad.jsonl", 8, 1, 0, tok, tok)


def test_embedding_dataset(tmp_path: Path, tok: Tokenizer):
    rec = {"query": ["find :", "cat"], "positives": [["doc :", "the cat sat"]], "negatives": [["doc :", "a dog ran"]]}
    (tmp_path / "emb.jsonl").write_text(json.dumps(rec) + "\n")
    ds = EmbeddingDataset(tmp_path / "emb.jsonl", sequence_length=8, seed=1, tokenizer=tok, number_of_hard_negatives=1)
    item = ds[0]
    assert item.input_token_ids.shape == (3, 8)
    q = tok.encode("find : cat")
    assert item.input_token_ids[0].tolist()[:len(q)] == q
    assert item.loss_weights[0].tolist() == [0, 0, 1] + [0] * 5  # instruction and padding are not pooled
    batch = ds.collate([item, item])
    assert batch.input_token_ids.shape == (6, 8)
    no_instr = EmbeddingDataset(tmp_path / "emb.jsonl", 8, 1, tok, 1, use_instruction=False)
    assert no_instr[0].input_token_ids[0].tolist()[:1] == tok.encode("cat")
    EmbeddingDataset.jsonl_to_embedding_mmap(tmp_path / "emb.jsonl", tok, tmp_path / "embmap")
    mm = EmbeddingDataset(tmp_path / "embmap", 8, 1, tok, 1, memory_map_dataset=True)
    assert torch.equal(mm[0].input_token_ids, item.input_token_ids)
    assert torch.equal(mm[0].loss_weights, item.loss_weights)
    with pytest.raises(NotImplementedError):
        EmbeddingDataset(tmp_path / "emb.jsonl", 8, 1, tok, 2)


def test_tokenizer_variants(tmp_path: Path, tok: Tokenizer):
    assert tok.decode(tok.encode("the cat")) == "the cat"
    assert tok.eos_token_id == tok.padding_token_id == 0
    definition = json.loads(tok.tokenizer.to_str())
    definition["pre_tokenizer"] = {"type": "ByteLevel", "add_prefix_space": True, "trim_offsets": True, "use_regex": True}
    (tmp_path / "vocab.json").write_text(json.dumps(definition))
    plain, no_space = load_tokenizers(tmp_path / "vocab.json")
    assert plain is not no_space
    (tmp_path / "plain.json").write_text(tok.tokenizer.to_str())
    a, b = load_tokenizers(tmp_path / "plain.json")
    assert a is b  # nothing to switch off


def test_samplers():
    torch.manual_seed(0)
    logits = torch.tensor([[[0.0, 1.0, 5.0, 2.0], [3.0, 0.5, 0.1, 0.2]]])
    assert sample_argmax(logits).tolist() == [0]
    k = top_k_transform(logits, k=2)
    assert torch.isinf(k[0, 0, 0]) and torch.isinf(k[0, 0, 1]) and not torch.isinf(k[0, 0, 2])
    p = top_p_transform(logits, threshold=0.5)
    assert not torch.isinf(p[0, 0, 2]) and torch.isinf(p[0, 0, 0])  # the top token alone carries > 50 %
    draws = torch.stack([sample_temperature(logits, 0.01) for _ in range(20)])
    assert (draws == 0).all()  # near-zero temperature = argmax


def test_pb_memory_map_and_text_image_dataset(tmp_path: Path, tok: Tokenizer):
    from io import BytesIO

    from PIL import Image

    from scaling_b200.core.data import PbMemoryMap, PbMemoryMapBuilder
    from scaling_b200.transformer.data import TextImageDataset

    img = tmp_path / "x.png"
    Image.new("RGB", (40, 30), (200, 10, 10)).save(img)
    b = PbMemoryMapBuilder(tmp_path / "ti", tokenizer=tok, tokenizer_no_prefix_space=tok, image_encoder_token_counts=4)
    b.add([{"type": "image", "content": str(img)}, {"type": "text", "content": "the cat", "has_loss": False},
           {"type": "text", "content": "sat on", "has_loss": True}])
    b.add([{"type": "text", "content": "a dog ran far", "has_loss": True}])
    b.finalize()
    mm = PbMemoryMap(tmp_path / "ti")
    assert len(mm) == 2
    assert mm[0]["prompt_image_locations"] == [{"start_index": 0, "end_index": 4}]
    assert mm[0]["input_token_list"] == [0, 0, 0, 0] + tok.encode("the cat") + tok.encode("sat")
    assert Image.open(BytesIO(mm[0]["prompt_image_data"][0])).size == (40, 30)
    with pytest.raises(ValueError):
        PbMemoryMapBuilder(tmp_path / "ti")  # refuses to overwrite

    ds = TextImageDataset(tmp_path / "ti", sequence_length=10, softprompt_n_tokens=1, shuffle=False, seed=5)
    item = ds[0]
    assert item.input_image_locations == [(1, 5)]  # shifted by the soft prompt
    assert item.input_images[0].shape == (3, 384, 384)
    assert item.loss_weights.tolist() == [0, 0, 0, 0, 0, 0, 1, 1, 0, 0]
    batch = ds.collate([ds[0], ds[1]])
    assert batch.input_images.shape == (1, 3, 384, 384) and batch.input_image_locations.tolist() == [[0, 1, 5]]


def test_legacy_indexed_datasets(tmp_path: Path):
    from scaling_b200.transformer.data.legacy_dataset.indexed_dataset import (infer_dataset_impl, make_builder,
                                                                              make_dataset)

    docs = [np.arange(5), np.arange(3) + 10, np.array([7])]
    for impl in ("mmap", "cached"):
        prefix = str(tmp_path / impl)
        b = make_builder(prefix + ".bin", impl, vocab_size=1000)
        for d in docs:
            b.add_item(torch.tensor(d))
            if impl == "mmap":
                b.end_document()
        b.finalize(prefix + ".idx")
        assert infer_dataset_impl(prefix) == impl
        ds = make_dataset(prefix)
        assert [ds[i].tolist() for i in range(len(ds))] == [d.tolist() for d in docs]
    ds = make_dataset(str(tmp_path / "mmap"))
    assert ds.sizes.tolist() == [5, 3, 1] and ds.get(0, offset=1, length=2).tolist() == [1, 2]
    text = TextDataset(data_prefix=tmp_path / "mmap", sequence_length=4, seed=1, legacy_dataset=True)
    assert len(text) >= 1 and text[0].token_ids.numel() == 5


def test_text_windows_overlap_by_one_token_and_drop_the_tail():
    """Documents are walked in the given order; a window holds sequence_length + 1 tokens, its last token opens the
    next window, what cannot fill a window is dropped; `only_full_sequences` starts every window inside one document."""
    from scaling_b200.transformer.data.text_dataset import pack_windows

    sizes = [7, 3, 12]
    windows = pack_windows(sizes, doc_order=[0, 1, 2], sequence_length=4)
    triples = [w.reshape(-1, 3).tolist() for w in windows]
    flat = [[(d, i) for d, s, e in t for i in range(s, e)] for t in triples]
    assert all(len(f) == 5 for f in flat)
    for a, b in zip(flat, flat[1:]):
        assert a[-1] == b[0]  # the target of the last position is the input of the next window's first
    stream = [(d, i) for d in (0, 1, 2) for i in range(sizes[d])]
    covered = [flat[0][0]] + [p for f in flat for p in f[1:]]
    assert covered == stream[:len(covered)] and len(stream) - len(covered) < 4  # only a tail shorter than a window is lost
    full = pack_windows(sizes, doc_order=[0, 1, 2], sequence_length=4, only_full_sequences=True)
    for w in full:
        t = w.reshape(-1, 3).tolist()
        assert len(t) == 1 and t[0][2] - t[0][1] == 5  # one document per window, never a stitched one
    assert {w.reshape(-1, 3)[0][0] for w in full} == {0, 2}  # the 3-token document cannot fill a window


def test_sampler_indices_follow_the_consumed_samples():
    """epoch = consumed // usable, indices stride over the data-parallel ranks, the remainder of an epoch is cut."""
    from scaling_b200.core.data.dataloader import RandomSampler

    class _DS:
        def __len__(self):
            return 23

        def set_seed(self, seed, shuffle=True):
            self.seed = seed

    def batches(dp_rank, consumed, n):
        from types import SimpleNamespace

        ds = _DS()
        topology = SimpleNamespace(config=SimpleNamespace(micro_batch_size=2, data_parallel_size=2),
                                   data_parallel_rank=dp_rank)
        s = iter(RandomSampler(dataset=ds, seed=5, consumed_samples=consumed, topology=topology))
        out = [b for _, b in zip(range(n), s)]
        return out, ds.seed

    r0, seed0 = batches(0, 0, 99)
    r1, _ = batches(1, 0, 99)
    usable = (23 // 2 // 2) * 2 * 2  # 20 samples per epoch: five micro batches of two per rank
    assert len(r0) == len(r1) == 5 and seed0 == 5
    assert r0[0] == [0, 2] and r1[0] == [1, 3]
    assert sorted(i for b in r0 + r1 for i in b) == list(range(usable))
    resumed, seed = batches(0, 8, 99)
    assert resumed == r0[2:] and seed == 5
    wrapped, seed = batches(0, usable + 4, 1)
    assert wrapped == [r0[1]] and seed == 6  # the next epoch reshuffles the data with seed + epoch


def _legacy_corpus(prefix: Path, n_docs: int, doc_len: int, base: int) -> None:
    from scaling_b200.transformer.data.legacy_dataset.indexed_dataset import make_builder

    b = make_builder(str(prefix) + ".bin", "mmap", vocab_size=1000)
    for d in range(n_docs):
        b.add_item(torch.arange(doc_len) + base + d)
        b.end_document()
    b.finalize(str(prefix) + ".idx")


def test_legacy_blended_dataset_index_files_and_interleaving(tmp_path: Path):
    """The legacy blend writes `.bin/.idx/.done` under the legacy cache name, interleaves the sources by always taking
    from the dataset furthest below its target (checked against the plain loop), and a second instance reuses the files."""
    import hashlib

    from scaling_b200.core.data.blended_dataset_config import BlendedDatasetConfig
    from scaling_b200.transformer.data import LegacyBlendedDataset
    from scaling_b200.transformer.data.legacy_dataset.indexed_dataset import make_dataset

    _legacy_corpus(tmp_path / "small", n_docs=6, doc_len=9, base=1)
    _legacy_corpus(tmp_path / "large", n_docs=30, doc_len=9, base=500)
    seq = 4
    sets = [TextDataset(data_prefix=tmp_path / n, sequence_length=seq, seed=3, legacy_dataset=True) for n in ("small", "large")]
    cfg = BlendedDatasetConfig(weight_by_num_documents=True, weighted_sampler_alpha=0.5, cache_directory=tmp_path / "cache")
    blend = LegacyBlendedDataset(seed=3, config=cfg, datasets=sets)

    counts = [len(s) for s in sets]
    p = np.asarray(counts, dtype=np.float64) / sum(counts)
    q = p ** 0.5 / (p ** 0.5).sum()
    w = (q / p) / (q / p).sum()
    assert np.allclose(blend.weights, w)
    targets = np.array([max(1, int(x * n)) for n, x in zip(counts, w / w.max())], dtype=np.int64)
    sampled = np.zeros(2, dtype=np.int64)
    expected = []
    while (sampled < targets).all():
        i = int((sampled / targets).argmin())
        expected.append([i, int(sampled[i])])
        sampled[i] += 1
    stem = blend.get_data_index_cache_filename_stem(3)
    name = Path(stem).name
    prefix_hash = hashlib.md5("small-large".encode()).hexdigest()
    assert name.startswith(f"index_cache_blended_dataset_seed_3_seq_len_{seq}_prefix_{prefix_hash}_weights_")
    assert all(Path(stem + ext).is_file() for ext in (".bin", ".idx", ".done"))
    stored = make_dataset(stem, "mmap")
    assert stored.dtype == np.int32 and [stored[i].tolist() for i in range(len(stored))] == expected
    assert len(blend) == len(expected)
    for k in (0, 1, len(expected) - 1):
        d, j = expected[k]
        assert torch.equal(blend[k].token_ids, sets[d][j].token_ids)

    before = {ext: Path(stem + ext).stat().st_mtime_ns for ext in (".bin", ".idx", ".done")}
    again = LegacyBlendedDataset(seed=3, config=cfg, datasets=sets)
    assert {ext: Path(stem + ext).stat().st_mtime_ns for ext in before} == before and len(again) == len(blend)
    # a rate limit per dataset (keyed by the stem of its prefix) caps the large corpus only
    ep = BlendedDatasetConfig(weight_by_num_documents=True, weight_examples_proportional=True,
                              cache_directory=tmp_path / "cache_ep")
    capped = LegacyBlendedDataset(seed=3, config=ep, datasets=sets, ep_maximum_dict={"large": counts[0]})
    assert np.allclose(capped.weights * np.asarray(counts) / (capped.weights * np.asarray(counts)).sum(), [0.5, 0.5])
    single = LegacyBlendedDataset(seed=3, config=cfg, datasets=sets[:1])
    assert len(single) == counts[0] and torch.equal(single[2].token_ids, sets[0][2].token_ids)
