"""Model hub and packaging (``crates/torsh-hub``, ``crates/torsh-package``).

``LocalHub`` is a directory-backed registry (publish / fetch / list / search, versioned entries with SHA-256 integrity
and a JSON model card); remote download is refused when no network is reachable rather than silently skipped.
``Package`` is a torch.package-like archive: a zip with a manifest (name, version, dependencies, per-file SHA-256),
optional zlib compression and an HMAC-SHA256 signature over the manifest (the reference signs with ed25519, which
needs a library that is not in this image)."""
from __future__ import annotations

import hashlib
import hmac
import json
import shutil
import time
import zipfile
from pathlib import Path


def sha256_file(path) -> str:
    h = hashlib.sha256()
    with open(path, "rb") as f:
        for chunk in iter(lambda: f.read(1 << 20), b""):
            h.update(chunk)
    return h.hexdigest()


def default_hub_dir() -> Path:
    """``TORSH_HUB_DIR``, else ``TORSH_MODEL_CACHE``, else ``~/.cache/torsh/hub`` (the reference's environment names)."""
    import os
    return Path(os.environ.get("TORSH_HUB_DIR") or os.environ.get("TORSH_MODEL_CACHE") or Path.home() / ".cache" / "torsh" / "hub")


class LocalHub:
    def __init__(self, root=None):
        self.root = Path(root) if root is not None else default_hub_dir()
        self.root.mkdir(parents=True, exist_ok=True)
        self.index_path = self.root / "index.json"

    def _index(self) -> dict:
        return json.loads(self.index_path.read_text()) if self.index_path.exists() else {}

    def publish(self, name: str, path, version: str | None = None, card: dict | None = None) -> dict:
        idx = self._index()
        version = version or f"v{len(idx.get(name, {})) + 1}"
        dst = self.root / name.replace("/", "__") / version
        dst.mkdir(parents=True, exist_ok=True)
        f = dst / Path(path).name
        shutil.copyfile(path, f)
        entry = {"file": str(f.relative_to(self.root)), "sha256": sha256_file(f), "size": f.stat().st_size,
                 "published": time.time(), "card": card or {}}
        idx.setdefault(name, {})[version] = entry
        self.index_path.write_text(json.dumps(idx, indent=1))
        return {"name": name, "version": version, **entry}

    def list(self) -> list[str]:
        return [f"{n}@{v}" for n, vs in sorted(self._index().items()) for v in vs]

    def search(self, query: str) -> list[str]:
        q = query.lower()
        return [e for e in self.list() if q in e.lower()]

    def fetch(self, name: str, version: str | None = None, output=None) -> Path:
        idx = self._index()
        if name not in idx:
            if "://" in name or name.count("/") == 1:
                raise ConnectionError(f"{name!r} is not in the local hub and no network is reachable")
            raise KeyError(name)
        version = version or sorted(idx[name])[-1]
        e = idx[name][version]
        src = self.root / e["file"]
        if sha256_file(src) != e["sha256"]:
            raise IOError(f"integrity check failed for {name}@{version}")
        if output:
            Path(output).parent.mkdir(parents=True, exist_ok=True)
            shutil.copyfile(src, output)
            return Path(output)
        return src

    def load(self, name: str, version: str | None = None):
        """Fetch, decode and instantiate: the card's ``architecture`` names a registry entry."""
        from . import models
        from .serialize import model_state as ms
        st = ms.load_binary(self.fetch(name, version))
        m = models.create_model(st["metadata"]["architecture"])
        ms.load_model_state(m, st, strict=False)
        return m


def _ed25519_private(k):
    from cryptography.hazmat.primitives.asymmetric.ed25519 import Ed25519PrivateKey
    return k if isinstance(k, Ed25519PrivateKey) else Ed25519PrivateKey.from_private_bytes(bytes(k))


def _ed25519_public(k):
    from cryptography.hazmat.primitives.asymmetric.ed25519 import Ed25519PublicKey
    return k if isinstance(k, Ed25519PublicKey) else Ed25519PublicKey.from_public_bytes(bytes(k))


def generate_signing_key() -> tuple[bytes, bytes]:
    """New Ed25519 key pair as raw bytes ``(private 32 B, public 32 B)``."""
    from cryptography.hazmat.primitives import serialization as ser
    from cryptography.hazmat.primitives.asymmetric.ed25519 import Ed25519PrivateKey
    sk = Ed25519PrivateKey.generate()
    return (sk.private_bytes(ser.Encoding.Raw, ser.PrivateFormat.Raw, ser.NoEncryption()),
            sk.public_key().public_bytes(ser.Encoding.Raw, ser.PublicFormat.Raw))


def _seal(key: bytes, name: str, data: bytes) -> bytes:
    import os as _os
    from cryptography.hazmat.primitives.ciphers.aead import AESGCM
    nonce = _os.urandom(12)
    return nonce + AESGCM(key).encrypt(nonce, data, name.encode())          # the file name is authenticated too


def _open(key: bytes, name: str, blob: bytes) -> bytes:
    from cryptography.exceptions import InvalidTag
    from cryptography.hazmat.primitives.ciphers.aead import AESGCM
    try:
        return AESGCM(key).decrypt(blob[:12], blob[12:], name.encode())
    except InvalidTag:
        raise PermissionError(f"{name}: decryption failed (wrong key or modified data)") from None


class Package:
    MANIFEST = "MANIFEST.json"

    def __init__(self, name: str, version: str = "0.1.0", dependencies: dict | None = None):
        self.name, self.version, self.dependencies = name, version, dependencies or {}
        self.files: dict[str, bytes] = {}

    def add_bytes(self, arcname: str, data: bytes): self.files[arcname] = data
    def add_file(self, path, arcname: str | None = None): self.files[arcname or Path(path).name] = Path(path).read_bytes()
    def add_source(self, module_name: str, source: str): self.files[f"code/{module_name.replace('.', '/')}.py"] = source.encode()

    def add_model(self, model, arcname="model.trsm", architecture=None):
        from .serialize import model_state as ms
        self.files[arcname] = ms.encode_binary(ms.model_state(model, architecture=architecture))

    def manifest(self) -> dict:
        return {"name": self.name, "version": self.version, "dependencies": self.dependencies, "format": 1,
                "files": {k: {"sha256": hashlib.sha256(v).hexdigest(), "size": len(v)} for k, v in sorted(self.files.items())}}

    def save(self, path, compress: bool = True, key: bytes | None = None, signing_key=None,
             encryption_key: bytes | None = None) -> None:
        """``key``: shared secret for an HMAC-SHA256 signature. ``signing_key``: an Ed25519 private key (object or 32 raw
        bytes) for a public-key signature over the manifest (``crates/torsh-package``: ed25519). ``encryption_key``:
        16 / 24 / 32 bytes; file contents are sealed with AES-GCM (the manifest, which holds the plaintext hashes, is not)."""
        man_d = self.manifest()
        man_d["encrypted"] = encryption_key is not None
        man = json.dumps(man_d, sort_keys=True).encode()
        with zipfile.ZipFile(path, "w", zipfile.ZIP_DEFLATED if compress else zipfile.ZIP_STORED) as z:
            z.writestr(self.MANIFEST, man)
            if key is not None:
                z.writestr("SIGNATURE", hmac.new(key, man, hashlib.sha256).hexdigest())
            if signing_key is not None:
                z.writestr("SIGNATURE.ed25519", _ed25519_private(signing_key).sign(man))
            for k, v in self.files.items():
                z.writestr(k, _seal(encryption_key, k, v) if encryption_key is not None else v)

    @classmethod
    def load(cls, path, key: bytes | None = None, public_key=None, encryption_key: bytes | None = None) -> "Package":
        with zipfile.ZipFile(path) as z:
            man_raw = z.read(cls.MANIFEST)
            man = json.loads(man_raw)
            if key is not None:
                sig = z.read("SIGNATURE").decode() if "SIGNATURE" in z.namelist() else ""
                if not hmac.compare_digest(sig, hmac.new(key, man_raw, hashlib.sha256).hexdigest()):
                    raise PermissionError("package signature does not verify")
            if public_key is not None:
                from cryptography.exceptions import InvalidSignature
                if "SIGNATURE.ed25519" not in z.namelist():
                    raise PermissionError("package carries no Ed25519 signature")
                try:
                    _ed25519_public(public_key).verify(z.read("SIGNATURE.ed25519"), man_raw)
                except InvalidSignature:
                    raise PermissionError("package signature does not verify") from None
            if man.get("encrypted") and encryption_key is None:
                raise PermissionError("package is encrypted: an encryption key is needed")
            pkg = cls(man["name"], man["version"], man["dependencies"])
            for k, meta in man["files"].items():
                data = z.read(k)
                if man.get("encrypted"):
                    data = _open(encryption_key, k, data)
                if hashlib.sha256(data).hexdigest() != meta["sha256"]:
                    raise IOError(f"{k}: checksum mismatch")
                pkg.files[k] = data
        return pkg

    def import_module(self, module_name: str):
        import types
        src = self.files[f"code/{module_name.replace('.', '/')}.py"].decode()
        mod = types.ModuleType(module_name)
        exec(compile(src, f"<package {self.name}:{module_name}>", "exec"), mod.__dict__)
        return mod


def resolve_dependencies(requirements: dict[str, str], available: dict[str, list[str]]) -> dict[str, str]:
    """Pick the highest available version satisfying each ``>=x`` / ``==x`` / ``^x`` requirement."""
    key = lambda v: tuple(int(p) for p in v.split("."))
    out = {}
    for name, req in requirements.items():
        cands = sorted(available.get(name, []), key=key)
        if req.startswith("=="):
            ok = [v for v in cands if v == req[2:]]
        elif req.startswith(">="):
            ok = [v for v in cands if key(v) >= key(req[2:])]
        elif req.startswith("^"):
            base = key(req[1:])
            ok = [v for v in cands if key(v) >= base and key(v)[0] == base[0]]
        else:
            ok = cands
        if not ok:
            raise LookupError(f"no version of {name} satisfies {req!r} (have {cands})")
        out[name] = ok[-1]
    return out


# -------------------------------------------------------------------------------------- Hugging Face checkpoint import
_HF_GPT2_TRANSPOSED = ("attn.c_attn.weight", "attn.c_proj.weight", "mlp.c_fc.weight", "mlp.c_proj.weight")


def import_hf_gpt2(hf_state: dict, model) -> list[str]:
    """Copy a Hugging Face GPT-2 ``state_dict`` into a :class:`torsh_b200.models.GPTForCausalLM`
    (``crates/torsh-hub``: Hugging Face integration). HF stores the four projection weights of a block as ``Conv1D``
    (``[in, out]``) and the embeddings as ``wte.weight`` / ``wpe.weight``; here linear weights are ``[out, in]`` and the
    embeddings are plain parameters. Returns the HF keys that were not used (attention-mask buffers, a tied ``lm_head``)."""
    import torch
    own = dict(model.named_parameters())
    used = set()
    with torch.no_grad():
        for name, p in own.items():
            key = name + ".weight" if name in ("transformer.wte", "transformer.wpe") else name
            if key not in hf_state:
                raise KeyError(f"checkpoint has no tensor for {name!r} (looked for {key!r})")
            src = hf_state[key]
            if name.endswith(_HF_GPT2_TRANSPOSED):
                src = src.t()
            if name == "transformer.wte" and src.shape[0] < p.shape[0]:       # vocabulary padded to a tile multiple
                p[: src.shape[0]].copy_(src.to(p.dtype))
            else:
                if tuple(src.shape) != tuple(p.shape):
                    raise ValueError(f"{name}: checkpoint shape {tuple(src.shape)} != model shape {tuple(p.shape)}")
                p.copy_(src.to(p.dtype))
            used.add(key)
    return sorted(k for k in hf_state if k not in used)


class AccessControl:
    """Token-based access to hub entries (``crates/torsh-hub``: access control): tokens are stored as SHA-256 digests
    with a role (``read`` / ``write`` / ``admin``) and optional name prefixes; the environment variable
    ``TORSH_HUB_TOKEN`` supplies the caller's token when none is passed."""

    ROLES = {"read": 1, "write": 2, "admin": 3}

    def __init__(self, path=None):
        self.path = Path(path) if path else None
        self.tokens: dict[str, dict] = json.loads(self.path.read_text()) if self.path and self.path.exists() else {}

    def _save(self):
        if self.path:
            self.path.write_text(json.dumps(self.tokens, indent=1))

    @staticmethod
    def _digest(token: str) -> str:
        return hashlib.sha256(token.encode()).hexdigest()

    def grant(self, token: str, role: str = "read", prefixes: tuple[str, ...] = ("",)):
        if role not in self.ROLES:
            raise ValueError(f"unknown role {role!r}")
        self.tokens[self._digest(token)] = {"role": role, "prefixes": list(prefixes)}
        self._save()

    def revoke(self, token: str):
        self.tokens.pop(self._digest(token), None)
        self._save()

    def allowed(self, action: str, name: str, token: str | None = None) -> bool:
        import os
        token = token if token is not None else os.environ.get("TORSH_HUB_TOKEN", "")
        e = self.tokens.get(self._digest(token))
        if e is None:
            return False
        return self.ROLES[e["role"]] >= self.ROLES[action] and any(name.startswith(p) for p in e["prefixes"])

    def require(self, action: str, name: str, token: str | None = None):
        if not self.allowed(action, name, token):
            raise PermissionError(f"token may not {action} {name!r}")


def import_hf_llama(hf_state: dict, model) -> list[str]:
    """Copy a Hugging Face Llama ``state_dict`` (multi-head attention, no grouped KV) into a
    :class:`torsh_b200.models.LlamaModel` built without tensor parallelism. Three layout differences are bridged:
    the fused ``qkv`` (``[q | k | v]``) and ``gate_up`` (``[up | gate]``: the gate is the second half) projections, and
    the rotary convention — HF rotates the pairs ``(i, i + D/2)`` of a head, this package the adjacent pairs
    ``(2i, 2i + 1)`` — so the rows of the query and key projections are interleaved per head. Returns unused HF keys."""
    import torch
    cfg = model.cfg
    E, H, D = cfg.hidden_size, cfg.num_heads, cfg.head_dim

    def interleave(w):                                    # [H*D, E] rows (i, i + D/2) -> (2i, 2i + 1) inside every head
        return w.view(H, 2, D // 2, E).transpose(1, 2).reshape(H * D, E)

    used = set()

    def take(key):
        if key not in hf_state:
            raise KeyError(f"checkpoint has no tensor {key!r}")
        used.add(key)
        return hf_state[key]

    with torch.no_grad():
        emb = take("model.embed_tokens.weight")
        model.embed[: emb.shape[0]].copy_(emb.to(model.embed.dtype))
        for i, blk in enumerate(model.layers):
            pre = f"model.layers.{i}."
            if take(pre + "self_attn.k_proj.weight").shape[0] != E:
                raise ValueError("grouped-query attention checkpoints are not supported by this importer")
            q, k, v = (take(pre + f"self_attn.{n}_proj.weight") for n in ("q", "k", "v"))
            blk.qkv.weight.copy_(torch.cat([interleave(q), interleave(k), v]).to(blk.qkv.weight.dtype))
            blk.o.weight.copy_(take(pre + "self_attn.o_proj.weight").to(blk.o.weight.dtype))
            blk.gate_up.weight.copy_(torch.cat([take(pre + "mlp.up_proj.weight"), take(pre + "mlp.gate_proj.weight")]).to(blk.gate_up.weight.dtype))
            blk.down.weight.copy_(take(pre + "mlp.down_proj.weight").to(blk.down.weight.dtype))
            blk.input_norm.weight.copy_(take(pre + "input_layernorm.weight").to(blk.input_norm.weight.dtype))
            blk.post_attn_norm.weight.copy_(take(pre + "post_attention_layernorm.weight").to(blk.post_attn_norm.weight.dtype))
        model.norm.weight.copy_(take("model.norm.weight").to(model.norm.weight.dtype))
        head = hf_state.get("lm_head.weight", emb)
        used.add("lm_head.weight")
        model.lm_head[: head.shape[0]].copy_(head.to(model.lm_head.dtype))
    return sorted(k for k in hf_state if k not in used)


def import_hf_bert(hf_state: dict, model) -> list[str]:
    """Copy a Hugging Face ``BertModel`` ``state_dict`` into :class:`torsh_b200.models.BertModel` (post-norm encoder with a
    fused ``in_proj`` for query / key / value). Returns the HF keys that were not used (position-id buffers)."""
    import torch
    used = set()

    def take(key):
        if key not in hf_state:
            raise KeyError(f"checkpoint has no tensor {key!r}")
        used.add(key)
        return hf_state[key]

    def put(dst, *keys):
        src = torch.cat([take(k) for k in keys]) if len(keys) > 1 else take(keys[0])
        if tuple(src.shape) != tuple(dst.shape):
            raise ValueError(f"{keys[0]}: checkpoint shape {tuple(src.shape)} != model shape {tuple(dst.shape)}")
        dst.copy_(src.to(dst.dtype))

    with torch.no_grad():
        e = "embeddings."
        put(model.word_embeddings.weight, e + "word_embeddings.weight")
        pos = take(e + "position_embeddings.weight")
        model.position_embeddings.weight[: pos.shape[0]].copy_(pos)
        put(model.token_type_embeddings.weight, e + "token_type_embeddings.weight")
        put(model.emb_norm.weight, e + "LayerNorm.weight")
        put(model.emb_norm.bias, e + "LayerNorm.bias")
        for i, layer in enumerate(model.layers):
            p = f"encoder.layer.{i}."
            a = p + "attention.self."
            put(layer.attn.in_proj_weight, a + "query.weight", a + "key.weight", a + "value.weight")
            put(layer.attn.in_proj_bias, a + "query.bias", a + "key.bias", a + "value.bias")
            for ours, theirs in ((layer.attn.out_proj, "attention.output.dense"), (layer.ln1, "attention.output.LayerNorm"),
                                 (layer.fc1, "intermediate.dense"), (layer.fc2, "output.dense"), (layer.ln2, "output.LayerNorm")):
                put(ours.weight, p + theirs + ".weight")
                put(ours.bias, p + theirs + ".bias")
        if hasattr(model, "pooler") and "pooler.dense.weight" in hf_state:
            put(model.pooler.weight, "pooler.dense.weight")
            put(model.pooler.bias, "pooler.dense.bias")
    return sorted(k for k in hf_state if k not in used)


def import_hf_vit(hf_state: dict, model) -> list[str]:
    """Copy a Hugging Face ``ViTForImageClassification`` ``state_dict`` into :class:`torsh_b200.models.VisionTransformer`
    (pre-norm blocks, fused query / key / value projection)."""
    import torch
    used = set()

    def take(key):
        if key not in hf_state:
            raise KeyError(f"checkpoint has no tensor {key!r}")
        used.add(key)
        return hf_state[key]

    def put(dst, *keys):
        src = torch.cat([take(k) for k in keys]) if len(keys) > 1 else take(keys[0])
        if tuple(src.shape) != tuple(dst.shape):
            raise ValueError(f"{keys[0]}: checkpoint shape {tuple(src.shape)} != model shape {tuple(dst.shape)}")
        dst.copy_(src.to(dst.dtype))

    with torch.no_grad():
        e = "vit.embeddings."
        put(model.cls_token, e + "cls_token")
        put(model.pos_embed, e + "position_embeddings")
        put(model.patch_embed.weight, e + "patch_embeddings.projection.weight")
        put(model.patch_embed.bias, e + "patch_embeddings.projection.bias")
        for i, b in enumerate(model.blocks):
            p = f"vit.encoder.layer.{i}."
            a = p + "attention.attention."
            put(b.attn.in_proj_weight, a + "query.weight", a + "key.weight", a + "value.weight")
            put(b.attn.in_proj_bias, a + "query.bias", a + "key.bias", a + "value.bias")
            for ours, theirs in ((b.attn.out_proj, "attention.output.dense"), (b.ln1, "layernorm_before"),
                                 (b.fc1, "intermediate.dense"), (b.fc2, "output.dense"), (b.ln2, "layernorm_after")):
                put(ours.weight, p + theirs + ".weight")
                put(ours.bias, p + theirs + ".bias")
        put(model.norm.weight, "vit.layernorm.weight")
        put(model.norm.bias, "vit.layernorm.bias")
        put(model.head.weight, "classifier.weight")
        put(model.head.bias, "classifier.bias")
    return sorted(k for k in hf_state if k not in used)


def _hf_copier(hf_state: dict):
    """``(take, put, unused)`` helpers shared by the Hugging Face importers below."""
    import torch
    used = set()

    def take(key):
        if key not in hf_state:
            raise KeyError(f"checkpoint has no tensor {key!r}")
        used.add(key)
        return hf_state[key]

    def put(dst, *keys, zero_missing: bool = False):
        parts = []
        for k in keys:
            if zero_missing and k not in hf_state:
                parts.append(None)
            else:
                parts.append(take(k))
        if any(p is None for p in parts):
            n = dst.shape[0] // len(parts)
            parts = [torch.zeros(n, *dst.shape[1:], dtype=dst.dtype) if p is None else p for p in parts]
        src = torch.cat(parts) if len(parts) > 1 else parts[0]
        if tuple(src.shape) != tuple(dst.shape):
            raise ValueError(f"{keys[0]}: checkpoint shape {tuple(src.shape)} != model shape {tuple(dst.shape)}")
        dst.copy_(src.to(dst.dtype))

    return take, put, lambda: sorted(k for k in hf_state if k not in used)


def _put_attention_block(put, block, p: str, attn: str, ln1: str, fc1: str, fc2: str, ln2: str, q="q_proj", k="k_proj", v="v_proj",
                         out="out_proj"):
    a = p + attn + "."
    put(block.attn.in_proj_weight, a + q + ".weight", a + k + ".weight", a + v + ".weight")
    put(block.attn.in_proj_bias, a + q + ".bias", a + k + ".bias", a + v + ".bias", zero_missing=True)   # Whisper keys have no bias
    for ours, theirs in ((block.attn.out_proj, attn + "." + out), (block.ln1, ln1), (block.fc1, fc1), (block.fc2, fc2), (block.ln2, ln2)):
        put(ours.weight, p + theirs + ".weight")
        put(ours.bias, p + theirs + ".bias")


def import_hf_clip(hf_state: dict, model) -> list[str]:
    """Copy a Hugging Face ``CLIPModel`` ``state_dict`` into :class:`torsh_b200.models.multimodal.CLIPModel`."""
    import torch
    take, put, unused = _hf_copier(hf_state)
    with torch.no_grad():
        v, t = "vision_model.", "text_model."
        put(model.vision.patch_embed.weight, v + "embeddings.patch_embedding.weight")
        put(model.vision.class_embedding, v + "embeddings.class_embedding")
        put(model.vision.position_embedding, v + "embeddings.position_embedding.weight")
        for ours, theirs in ((model.vision.pre_ln, "pre_layrnorm"), (model.vision.post_ln, "post_layernorm")):
            put(ours.weight, v + theirs + ".weight"); put(ours.bias, v + theirs + ".bias")
        for i, b in enumerate(model.vision.layers):
            _put_attention_block(put, b, f"{v}encoder.layers.{i}.", "self_attn", "layer_norm1", "mlp.fc1", "mlp.fc2", "layer_norm2")
        put(model.text.token_embedding.weight, t + "embeddings.token_embedding.weight")
        put(model.text.position_embedding, t + "embeddings.position_embedding.weight")
        for i, b in enumerate(model.text.layers):
            _put_attention_block(put, b, f"{t}encoder.layers.{i}.", "self_attn", "layer_norm1", "mlp.fc1", "mlp.fc2", "layer_norm2")
        put(model.text.final_ln.weight, t + "final_layer_norm.weight"); put(model.text.final_ln.bias, t + "final_layer_norm.bias")
        put(model.visual_projection.weight, "visual_projection.weight")
        put(model.text_projection.weight, "text_projection.weight")
        put(model.logit_scale, "logit_scale")
    return [k for k in unused() if not k.endswith("position_ids")]


def import_hf_whisper_encoder(hf_state: dict, encoder, prefix: str = "encoder.") -> list[str]:
    """Copy the encoder of a Hugging Face ``WhisperModel`` into :class:`torsh_b200.models.audio.WhisperEncoder`. The key
    projection of Whisper has no bias; the fused ``in_proj_bias`` gets zeros there. Returns unused encoder keys."""
    import torch
    sub = {k[len(prefix):]: v for k, v in hf_state.items() if k.startswith(prefix)}
    take, put, unused = _hf_copier(sub)
    with torch.no_grad():
        for ours, theirs in ((encoder.conv1, "conv1"), (encoder.conv2, "conv2"), (encoder.ln_post, "layer_norm")):
            put(ours.weight, theirs + ".weight"); put(ours.bias, theirs + ".bias")
        put(encoder.embed_positions, "embed_positions.weight")
        for i, b in enumerate(encoder.layers):
            _put_attention_block(put, b, f"layers.{i}.", "self_attn", "self_attn_layer_norm", "fc1", "fc2", "final_layer_norm")
    return unused()


def import_hf_wav2vec2(hf_state: dict, model) -> list[str]:
    """Copy a Hugging Face ``Wav2Vec2Model`` ``state_dict`` into :class:`torsh_b200.models.audio.Wav2Vec2Model`. The
    positional convolution is stored weight-normalised (magnitude ``g`` per kernel position and direction ``v``); the
    effective weight ``g * v / ||v||`` is materialised here. Quantizer / masking tensors of the pre-training head are
    returned as unused."""
    import torch
    take, put, unused = _hf_copier(hf_state)
    with torch.no_grad():
        fe = "feature_extractor.conv_layers."
        for i, conv in enumerate(model.feature_extractor.convs):
            put(conv.weight, f"{fe}{i}.conv.weight")
            if conv.bias is not None:
                put(conv.bias, f"{fe}{i}.conv.bias")
        for i, nrm in enumerate(model.feature_extractor.norms):
            put(nrm.weight, f"{fe}{i}.layer_norm.weight"); put(nrm.bias, f"{fe}{i}.layer_norm.bias")
        put(model.feat_norm.weight, "feature_projection.layer_norm.weight"); put(model.feat_norm.bias, "feature_projection.layer_norm.bias")
        put(model.feat_proj.weight, "feature_projection.projection.weight"); put(model.feat_proj.bias, "feature_projection.projection.bias")
        pc = "encoder.pos_conv_embed.conv."
        if pc + "parametrizations.weight.original0" in hf_state:
            g, v = take(pc + "parametrizations.weight.original0"), take(pc + "parametrizations.weight.original1")
        else:
            g, v = take(pc + "weight_g"), take(pc + "weight_v")
        model.pos_conv.weight.copy_(g * v / v.norm(dim=(0, 1), keepdim=True))      # weight norm over dim 2 (kernel position)
        put(model.pos_conv.bias, pc + "bias")
        put(model.enc_norm.weight, "encoder.layer_norm.weight"); put(model.enc_norm.bias, "encoder.layer_norm.bias")
        for i, b in enumerate(model.layers):
            _put_attention_block(put, b, f"encoder.layers.{i}.", "attention", "layer_norm", "feed_forward.intermediate_dense",
                                 "feed_forward.output_dense", "final_layer_norm")
    return unused()
