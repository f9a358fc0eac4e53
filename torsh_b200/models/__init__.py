"""Model zoo and registry (``crates/torsh-models/src/lib.rs:9-43``)."""
from .gpt2 import GPT2Config, GPT2LMHeadModel, GPT2Model, GPTForCausalLM
from .llama import LlamaConfig, LlamaForCausalLM, LlamaModel
from .resnet import BasicBlock, BottleneckBlock, ResNet, ResNetConfig, SEBlock
from .transformer_zoo import (BertConfig, BertForMaskedLM, BertForSequenceClassification, BertModel, EncoderBlock,
                              EncoderConfig, EncoderDecoderModel, RobertaModel, Seq2SeqConfig, T5Model, ViTConfig,
                              VisionTransformer)
from .vision_zoo import AlexNet, ConvNeXt, DenseNet, EfficientNet, MobileNetV2, SwinTransformer, VGG
from .audio import (HubertModel, Wav2Vec2Config, Wav2Vec2ForCTC, Wav2Vec2Model, WavLMModel, WhisperConfig, WhisperEncoder,
                    WhisperModel)
from .multimodal import ALIGNModel, CLIPConfig, CLIPModel, DualEncoder
from . import few_shot, fine_tuning, generative, model_utils, rl, video, vision_3d

_REGISTRY = {
    "gpt2-tiny": lambda **kw: GPTForCausalLM(GPT2Config.tiny(**kw)),
    "gpt2": lambda **kw: GPTForCausalLM(GPT2Config.small(**kw)),
    "gpt2-medium": lambda **kw: GPTForCausalLM(GPT2Config.medium(**kw)),
    "gpt2-large": lambda **kw: GPTForCausalLM(GPT2Config.large(**kw)),
    "gpt2-xl": lambda **kw: GPTForCausalLM(GPT2Config.xl(**kw)),
    "llama-7b": lambda **kw: LlamaModel(LlamaConfig.llama_7b(**kw)),
    "resnet18": lambda **kw: ResNet(ResNetConfig.resnet18(**kw)),
    "resnet34": lambda **kw: ResNet(ResNetConfig.resnet34(**kw)),
    "resnet50": lambda **kw: ResNet(ResNetConfig.resnet50(**kw)),
    "resnet101": lambda **kw: ResNet(ResNetConfig.resnet101(**kw)),
    "resnet152": lambda **kw: ResNet(ResNetConfig.resnet152(**kw)),
    "resnext50_32x4d": lambda **kw: ResNet(ResNetConfig.resnext50_32x4d(**kw)),
    "wide_resnet50_2": lambda **kw: ResNet(ResNetConfig.wide_resnet50_2(**kw)),
    "vit_b_16": lambda **kw: VisionTransformer(ViTConfig.vit_b_16(**kw)),
    "vit_l_16": lambda **kw: VisionTransformer(ViTConfig.vit_l_16(**kw)),
    "bert-base": lambda **kw: BertModel(BertConfig.bert_base(**kw)),
    "bert-large": lambda **kw: BertModel(BertConfig.bert_large(**kw)),
    "roberta-base": lambda **kw: BertModel(BertConfig.roberta_base(**kw)),
    "t5-base": lambda **kw: EncoderDecoderModel(Seq2SeqConfig(**kw)),
    "alexnet": lambda **kw: AlexNet(**kw),
    "vgg11": lambda **kw: VGG(11, **kw), "vgg16": lambda **kw: VGG(16, **kw), "vgg16_bn": lambda **kw: VGG(16, True, **kw),
    "vgg19": lambda **kw: VGG(19, **kw),
    "densenet121": lambda **kw: DenseNet((6, 12, 24, 16), **kw), "densenet169": lambda **kw: DenseNet((6, 12, 32, 32), **kw),
    "mobilenet_v2": lambda **kw: MobileNetV2(**kw),
    "efficientnet_b0": lambda **kw: EfficientNet(**kw),
    "convnext_tiny": lambda **kw: ConvNeXt((3, 3, 9, 3), (96, 192, 384, 768), **kw),
    "convnext_small": lambda **kw: ConvNeXt((3, 3, 27, 3), (96, 192, 384, 768), **kw),
    "swin_t": lambda **kw: SwinTransformer(96, (2, 2, 6, 2), (3, 6, 12, 24), **kw),
    "swin_s": lambda **kw: SwinTransformer(96, (2, 2, 18, 2), (3, 6, 12, 24), **kw),
    "wav2vec2-base": lambda **kw: Wav2Vec2Model(Wav2Vec2Config.base(**kw)),
    "wav2vec2-large": lambda **kw: Wav2Vec2Model(Wav2Vec2Config.large(**kw)),
    "hubert-base": lambda **kw: HubertModel(Wav2Vec2Config.base(**kw)),
    "whisper-tiny": lambda **kw: WhisperModel(WhisperConfig.tiny_en(**kw)),
    "whisper-base": lambda **kw: WhisperModel(WhisperConfig.base(**kw)),
    "whisper-small": lambda **kw: WhisperModel(WhisperConfig.small(**kw)),
    "clip-vit-b-32": lambda **kw: CLIPModel(CLIPConfig.vit_b_32()),
    "dqn": lambda **kw: rl.DQN(rl.DQNConfig(**kw)), "ppo": lambda **kw: rl.PPO(rl.PPOConfig(**kw)), "a3c": lambda **kw: rl.A3C(rl.A3CConfig(**kw)),
    "resnet3d_18": lambda **kw: video.ResNet3D(video.ResNet3DConfig(**kw)),
    "slowfast": lambda **kw: video.SlowFast(video.SlowFastConfig(**kw)),
    "video_transformer": lambda **kw: video.VideoTransformer(video.VideoTransformerConfig(**kw)),
    "vae": lambda **kw: generative.VAE(generative.VAEConfig(**kw)), "gan": lambda **kw: generative.GAN(generative.GANConfig(**kw)),
    "diffusion_unet": lambda **kw: generative.DiffusionUNet(generative.DiffusionConfig(**kw)),
    "cnn3d": lambda **kw: vision_3d.CNN3D(vision_3d.CNN3DConfig(**kw)),
    "pointnet": lambda **kw: vision_3d.PointNet(vision_3d.PointNetConfig(**kw)),
    "pointnet2": lambda **kw: vision_3d.PointNetPlusPlus(vision_3d.PointNetPlusPlusConfig(**kw)),
}


def list_models() -> list[str]:
    return sorted(_REGISTRY)


def create_model(name: str, **kw):
    if name not in _REGISTRY:
        raise KeyError(f"unknown model {name!r}; available: {list_models()}")
    return _REGISTRY[name](**kw)


def register_model(name: str, factory) -> None:
    _REGISTRY[name] = factory
