"""Host-side units: wire protocol, text streaming, incremental tokenisation, CPU placement, affinity."""

import random

import pytest

from b200serve.api import protocol
from b200serve.api.text import Detokenizer, StopMatcher
from b200serve.router import cpu_place, router


# ----------------------------------------------------------------------------- protocol
def test_parse_completion_forms():
    assert protocol.parse_completion({"prompt": "hi"}).prompt == "hi"
    assert protocol.parse_completion({"prompt": ["hi"]}).prompt == "hi"
    assert protocol.parse_completion({"prompt": [1, 2]}).prompt == [1, 2]
    assert protocol.parse_completion({"prompt": [[1, 2]]}).prompt == [1, 2]
    r = protocol.parse_completion({"prompt": "x", "stream": True, "stream_options": {"include_usage": True}})
    assert r.stream and r.include_usage and r.sampling.max_tokens == 16 and r.sampling.temperature == 1.0
    for bad in ({"prompt": ""}, {"prompt": 3}, {"prompt": "x", "n": 2}, {"prompt": "x", "echo": True},
                {"prompt": "x", "best_of": 2}, {"prompt": "x", "temperature": "hot"}, {"prompt": "x", "stop": 3},
                {"prompt": "x", "logit_bias": {"1": 2}}, {"prompt": "x", "suffix": "y"}, []):
        with pytest.raises(protocol.RequestError):
            protocol.parse_completion(bad)


def test_parse_chat_limits_and_tool_arguments():
    r = protocol.parse_chat({"messages": [{"role": "user", "content": "x"}], "max_completion_tokens": 5, "max_tokens": 9})
    assert r.sampling.max_tokens == 5 and not r.thinking
    r = protocol.parse_chat({"messages": [{"role": "user", "content": "x"}]})
    assert r.sampling.max_tokens is None  # rest of the context
    r = protocol.parse_chat({"messages": [{"role": "assistant", "content": "", "tool_calls": [
        {"function": {"name": "f", "arguments": "{\"a\": 1}"}}]}], "chat_template_kwargs": {"enable_thinking": True}})
    assert r.messages[0]["tool_calls"][0]["function"]["arguments"] == {"a": 1} and r.thinking
    with pytest.raises(protocol.RequestError):
        protocol.parse_chat({"messages": []})


def test_usage_and_error_bodies():
    u = protocol.Usage(10, 4, 3).body()
    assert u == {"prompt_tokens": 10, "completion_tokens": 3, "total_tokens": 13,
                 "prompt_tokens_details": {"cached_tokens": 4}}
    assert protocol.error_body("nope", 404)["error"]["type"] == "NotFoundError"
    env = protocol.Envelope("m", "chat.completion")
    assert protocol.chat_chunk(env, {"content": "a"}, 5, None, True)["choices"][0]["token_ids"] == [5]
    assert protocol.completion_chunk(protocol.Envelope("m", "text_completion"), "a", None, "stop", True)["choices"][0]["token_ids"] == []


# ----------------------------------------------------------------------------- text
class _ByteTok:
    """Tokens are single bytes; decoding a cut multi-byte character gives U+FFFD."""

    def decode(self, ids, skip_special_tokens=True):
        return bytes(ids).decode("utf-8", errors="replace")


def test_detokenizer_holds_back_partial_characters():
    text = "naïve café 日本語 ok"
    d = Detokenizer(_ByteTok())
    out = [d.push(b) for b in text.encode()]
    assert all("�" not in o for o in out)
    assert "".join(out) + d.flush() == text


def test_stop_matcher_withholds_and_cuts():
    m = StopMatcher(["END", "##"])
    got = "".join(m.push(c) for c in "hello E wor EN") + m.push("D tail")
    assert got == "hello E wor " and m.stopped and m.flush() == ""
    m = StopMatcher(["zzz"])
    assert m.push("ab") == "" and m.push("cd") == "ab" and m.flush() == "cd"
    assert StopMatcher([]).push("abc") == "abc"


def test_incremental_tokenizer_matches_full_encode(tmp_path):
    from b200serve.api.tokenizer import TextCodec
    from b200serve.models.tiny import build_tokenizer

    build_tokenizer(400).save_pretrained(str(tmp_path))
    codec = TextCodec(tmp_path)
    assert codec.encoder.enabled
    rng = random.Random(0)
    words = ["def", "main", "(", ")", ":", "\n", "    ", "return", " ", "x", "+", "1", "\n\n", "Question", "?", "<|im_end|>",
             "\n<|im_start|>user\n", "é", "日本"]
    text = ""
    for _ in range(40):
        text += "".join(rng.choice(words) for _ in range(rng.randint(5, 60)))
        ids = codec.encode(text)
        assert ids == codec.tok.encode(text, add_special_tokens=False)
    assert codec.encoder.stats["tokenize_reused_chars"] > 0


# ----------------------------------------------------------------------------- cpu placement
def _fake_sysfs(root, nodes=2, cores_per_node=8, smt=2, l3_cores=4):
    n_phys = nodes * cores_per_node
    for node in range(nodes):
        cpus = []
        for c in range(cores_per_node):
            phys = node * cores_per_node + c
            cpus += [phys + t * n_phys for t in range(smt)]
        d = root / f"sys/devices/system/node/node{node}"
        d.mkdir(parents=True)
        (d / "cpulist").write_text(cpu_place.format_cpu_list(cpus))
    for phys in range(n_phys):
        sibs = [phys + t * n_phys for t in range(smt)]
        grp0 = phys // l3_cores * l3_cores
        l3 = [g + t * n_phys for g in range(grp0, grp0 + l3_cores) for t in range(smt)]
        for cpu in sibs:
            base = root / f"sys/devices/system/cpu/cpu{cpu}"
            (base / "topology").mkdir(parents=True)
            (base / "cache/index3").mkdir(parents=True)
            (base / "topology/thread_siblings_list").write_text(cpu_place.format_cpu_list(sibs))
            (base / "cache/index3/shared_cpu_list").write_text(cpu_place.format_cpu_list(l3))
    for i, node in enumerate([0, 0, 1, 1]):
        d = root / f"sys/bus/pci/devices/0000:0{i}:00.0"
        d.mkdir(parents=True)
        (d / "numa_node").write_text(str(node))
    return list(range(n_phys * smt))


def test_cpu_lists_round_trip():
    assert cpu_place.parse_cpu_list("0-3,8,10-11") == [0, 1, 2, 3, 8, 10, 11]
    assert cpu_place.format_cpu_list([3, 1, 2, 8, 10, 11]) == "1-3,8,10-11"


def test_replica_slices_are_disjoint_near_their_gpus_and_avoid_cpu0(tmp_path):
    allowed = _fake_sysfs(tmp_path)
    topo = cpu_place.Topology.read(tmp_path, allowed=allowed, gpu_bdfs=[f"0000:0{i}:00.0" for i in range(4)])
    assert topo.gpu_nodes == [0, 0, 1, 1] and len(topo.physical_cores()) == 16
    slices = cpu_place.replica_slices(topo, [[0], [1], [2], [3]])
    seen = set()
    for s, node in zip(slices, [0, 0, 1, 1]):
        assert not (seen & set(s.cpus))
        seen |= set(s.cpus)
        assert all(topo.node_of[c] == node for c in s.cpus)
        assert len(s.rank_cpus) == 1 and s.rank_cpus[0] in s.cpus
    assert all(topo.l3_of[c] != topo.l3_of[0] for c in seen)  # CPU 0's L3 group left to the kernel
    two = cpu_place.replica_slices(topo, [[0, 1], [2, 3]])
    assert len(two[0].rank_cpus) == 2 and len(set(two[0].rank_cpus)) == 2


def test_small_machines_fall_back_to_all_cores(tmp_path):
    allowed = _fake_sysfs(tmp_path, nodes=1, cores_per_node=4, smt=1, l3_cores=4)
    topo = cpu_place.Topology.read(tmp_path, allowed=allowed)
    slices = cpu_place.replica_slices(topo, [[], []])
    assert all(s.cpus for s in slices) and not (set(slices[0].cpus) & set(slices[1].cpus))


# ----------------------------------------------------------------------------- router units
def test_layout_resolution():
    R = router.resolve_layout
    assert R(None, None, None, gpus=[]) is None
    assert R(2, None, None, gpus=[]) == [[], []]
    assert R(None, None, None, gpus=[0]) is None
    assert R(None, None, None, gpus=list(range(8))) == [[i] for i in range(8)]
    assert R(None, 2, None, gpus=list(range(8))) == [[0, 1], [2, 3], [4, 5], [6, 7]]
    assert R(2, 2, None, gpus=list(range(8))) == [[0, 1], [2, 3]]
    assert R(None, None, "0,1;4,5", gpus=list(range(8))) == [[0, 1], [4, 5]]
    assert R(None, 8, None, gpus=list(range(8))) is None
    with pytest.raises(ValueError):
        R(5, 2, None, gpus=list(range(8)))
    with pytest.raises(ValueError):
        R(None, None, "0,1;1,2", gpus=list(range(8)))
    assert router.device_env([2, 3]) == {"CUDA_VISIBLE_DEVICES": "2,3"}


def test_affinity_follows_growing_prompts_and_balances_new_sessions():
    a = router.Affinity(3)
    s1 = list(range(500))
    s2 = list(range(1000, 1400))
    r1 = a.route(router.affinity_key("/v1/completions", {"prompt": s1}))
    r2 = a.route(router.affinity_key("/v1/completions", {"prompt": s2}))
    assert r1 != r2  # the second session goes to an idle replica
    a.finish(r1)
    assert a.route(router.affinity_key("/v1/completions", {"prompt": s1 + list(range(77))})) == r1
    chat = [{"role": "user", "content": "a"}]
    r3 = a.route(router.affinity_key("/v1/chat/completions", {"messages": chat}))
    grown = chat + [{"role": "assistant", "content": "b"}, {"role": "user", "content": "c"}]
    assert a.route(router.affinity_key("/v1/chat/completions", {"messages": grown})) == r3
    text = "x" * 3000
    r4 = a.route(router.affinity_key("/v1/completions", {"prompt": text}))
    assert a.route(router.affinity_key("/v1/completions", {"prompt": text + " more"})) == r4
    assert a.routed_by_affinity == 3


def test_direct_decode_matches_the_tokenizer_wrapper(tmp_path):
    """The detokenizer's shortcut through the tokenizer's backend gives the wrapper's text, streamed or whole."""
    import random

    from b200serve.api.text import Detokenizer, decoder_of
    from b200serve.api.tokenizer import TextCodec
    from b200serve.models.tiny import write_tiny_checkpoint

    write_tiny_checkpoint(tmp_path)
    tok = TextCodec(tmp_path).tok
    dec = decoder_of(tok)
    assert dec is decoder_of(tok)  # chosen once per tokenizer
    rng = random.Random(1)
    ids = [rng.randrange(0, len(tok)) for _ in range(1500)]
    for i in range(0, 1400, 37):
        assert dec(ids[i : i + 9]) == tok.decode(ids[i : i + 9], skip_special_tokens=True)
    det = Detokenizer(tok)
    parts = [det.push(t) for t in ids] + [det.flush()]
    assert "".join(parts) == tok.decode(ids, skip_special_tokens=True)

    class Odd:  # a tokenizer whose wrapper post-processes the text: the shortcut must not be taken
        clean_up_tokenization_spaces = True
        backend_tokenizer = tok.backend_tokenizer

        def decode(self, ids, skip_special_tokens=True):
            return tok.decode(ids, skip_special_tokens=skip_special_tokens).replace(" ", "_")

        def __len__(self):
            return len(tok)

    odd = Odd()
    assert decoder_of(odd)(ids[:8]) == odd.decode(ids[:8])
