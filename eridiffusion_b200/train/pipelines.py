"""Per-architecture training pipelines and the staged step orchestrator.

Reference (crates/training/src/pipelines/): ``TrainingPipeline`` trait (``prepare_batch,
encode_prompts, encode_images, add_noise, compute_loss, get_model_inputs, apply_snr_weight,
get_scheduler_config``; base_pipeline.rs:91-158), ``PromptEmbeds{with_pooled, with_mask, concat}``
(:160-198), ``PipelineUtils::{apply_noise_offset, apply_input_perturbation}`` (:201-222),
``FluxPipeline`` (flux_pipeline.rs: dynamic shift, guidance 1.0 while training, packed latents),
``SDXLPipeline`` (sdxl_pipeline.rs: eps / v / sample targets, min-SNR, time ids), ``SD3Pipeline``
(sd3_pipeline.rs: flow target, CLIP-L + CLIP-G + T5 concatenation), ``SD15Pipeline``
(sd15_pipeline.rs), ``PipelineFactory::create`` (mod.rs:30-64). And the staged executor
(crates/training/src/pipeline/{stages,orchestrator,adapter}.rs): ``StageName`` list, ``Ctx`` and an
``Orchestrator`` that runs an adapter's recipe stage by stage.

The ``Trainer`` already fuses noise + target + patchify into one kernel and loss + gradient into
another; the classes here are the reference's API shape over those same pieces, for callers that
drive a step themselves (custom loops, evaluation, prior-preservation mixes). Every pipeline
answers with an ``objective`` from ``objectives/`` so that training, validation and these calls
use one definition of the noise schedule.
"""
from __future__ import annotations

import enum
from dataclasses import dataclass, field

import torch

from ..data.augmentation import input_perturbation, noise_offset
from ..objectives import DDPM, FlowMatching, loss_fn


# ---------------------------------------------------------------------------- data carriers
@dataclass
class PromptEmbeds:
    encoder_hidden_states: torch.Tensor                    # [B, T, D]
    pooled_projections: torch.Tensor | None = None         # [B, P]
    attention_mask: torch.Tensor | None = None             # [B, T]

    @classmethod
    def with_pooled(cls, hidden, pooled):
        return cls(hidden, pooled)

    def with_mask(self, mask):
        self.attention_mask = mask
        return self

    def concat(self, other: "PromptEmbeds") -> "PromptEmbeds":
        """Batch-wise concatenation (e.g. conditional + unconditional); a missing mask counts as
        all ones when the other side has one."""
        def cat(a, b):
            return None if a is None and b is None else torch.cat([a, b], 0)
        ma, mb = self.attention_mask, other.attention_mask
        if (ma is None) != (mb is None):
            ma = ma if ma is not None else torch.ones(self.encoder_hidden_states.shape[:2], device=mb.device, dtype=mb.dtype)
            mb = mb if mb is not None else torch.ones(other.encoder_hidden_states.shape[:2], device=ma.device, dtype=ma.dtype)
        if (self.pooled_projections is None) != (other.pooled_projections is None):
            raise ValueError("cannot concatenate embeddings with and without a pooled vector")
        return PromptEmbeds(torch.cat([self.encoder_hidden_states, other.encoder_hidden_states], 0),
                            cat(self.pooled_projections, other.pooled_projections), cat(ma, mb))


@dataclass
class PreparedBatch:
    latents: torch.Tensor
    prompt: PromptEmbeds
    extras: dict = field(default_factory=dict)             # time_ids, grid_hw, grid_fhw, control ...
    loss_mask: torch.Tensor | None = None

    def as_dict(self):
        d = {"latents": self.latents, "txt": self.prompt.encoder_hidden_states, **self.extras}
        if self.prompt.pooled_projections is not None:
            d["pooled"] = self.prompt.pooled_projections
        return d


@dataclass
class PipelineConfig:
    prediction_type: str = "epsilon"        # epsilon | v | sample (DDPM families)
    loss: str = "mse"                       # mse | l1 | huber
    min_snr_gamma: float | None = None
    noise_offset: float = 0.0
    input_perturbation: float = 0.0
    zero_terminal_snr: bool = False
    timestep_sampler: str = "logit_normal"  # flow families
    dynamic_shift: bool = True              # FLUX: resolution-dependent timestep shift
    guidance: float = 1.0                   # value fed to a guidance embedder while training
    snr_sqrt_weighting: bool = False        # SD3.5 optional weight sqrt(snr / (1 + snr))
    patch: int = 2


# ---------------------------------------------------------------------------- pipelines
class TrainingPipeline:
    architecture = "generic"
    patch = 2

    def __init__(self, config: PipelineConfig | None = None):
        self.config = config or PipelineConfig()
        self.objective = self._objective()

    def _objective(self):
        raise NotImplementedError

    # -- batch / conditioning
    def prepare_batch(self, batch: dict) -> PreparedBatch:
        extras = {k: v for k, v in batch.items() if k not in ("latents", "txt", "pooled", "mask", "loss_mask")}
        return PreparedBatch(batch["latents"], PromptEmbeds(batch["txt"], batch.get("pooled"), batch.get("mask")),
                             extras, batch.get("loss_mask"))

    def encode_prompts(self, prompts, encoders) -> PromptEmbeds:
        """``encoders``: callable(s) ``prompts -> (hidden [B, T, D], pooled or None)``."""
        hidden, pooled = encoders(prompts)
        return PromptEmbeds(hidden, pooled)

    def encode_images(self, images, vae):
        return vae.encode(images)

    # -- noise
    def sample_timesteps(self, n, gen=None, device="cpu"):
        return self.objective.sample_t(n, gen, device)

    def make_noise(self, latents, gen=None):
        # drawn on the generator's device (a CPU generator gives the same noise on every back end)
        eps = torch.randn(latents.shape, generator=gen, device=latents.device if gen is None else gen.device)
        eps = eps.to(latents.device)
        c = self.config
        if c.noise_offset:
            eps = noise_offset(eps, c.noise_offset, gen)
        if c.input_perturbation:
            eps = input_perturbation(eps, c.input_perturbation, gen)
        return eps.to(latents.dtype)

    def add_noise(self, latents, noise, timesteps):
        """Noisy latents and the regression target, in latent layout."""
        a, s, ca, cb = (r.view(-1, *([1] * (latents.dim() - 1))) for r in self.objective.coefficients(timesteps))
        lf, nf = latents.float(), noise.float()
        return (a * lf + s * nf).to(latents.dtype), (ca * nf + cb * lf).to(latents.dtype)

    # -- model call and loss
    def get_model_inputs(self, noisy_latents, timesteps, prompt: PromptEmbeds, batch: PreparedBatch) -> dict:
        raise NotImplementedError

    def call_model(self, model, inputs: dict):
        return model(**inputs)

    def postprocess_outputs(self, out, batch: PreparedBatch):
        return out

    def apply_snr_weight(self, timesteps):
        return self.objective.loss_weight(timesteps)

    def compute_loss(self, model, noisy_latents, target, timesteps, prompt: PromptEmbeds, batch: PreparedBatch):
        pred = self.postprocess_outputs(self.call_model(model, self.get_model_inputs(noisy_latents, timesteps, prompt,
                                                                                    batch)), batch)
        tgt = self.pack(target)
        if batch.loss_mask is not None:
            m = self.pack(batch.loss_mask.expand_as(target).to(pred.dtype))
            pred, tgt = pred * m, tgt * m
        return loss_fn(self.config.loss, pred, tgt, self.apply_snr_weight(timesteps))

    def compute_prior_loss(self, model, prior_batch: dict | None, gen=None):
        """Prior-preservation term: the same loss on a batch of class images (None when unused)."""
        if prior_batch is None:
            return None
        return self.training_loss(model, prior_batch, gen)

    def training_loss(self, model, batch: dict, gen=None):
        pb = self.prepare_batch(batch)
        t = self.sample_timesteps(pb.latents.shape[0], gen, pb.latents.device)
        noisy, target = self.add_noise(pb.latents, self.make_noise(pb.latents, gen), t)
        return self.compute_loss(model, noisy, target, t, pb.prompt, pb)

    def pack(self, x):
        """Latent layout -> the layout of the model's prediction."""
        return x

    def get_scheduler_config(self) -> dict:
        o = self.objective
        return {k: v for k, v in vars(o).items() if isinstance(v, (int, float, str, bool, type(None)))}


def _patchify(x, p):
    B, C, H, W = x.shape
    return x.view(B, C, H // p, p, W // p, p).permute(0, 2, 4, 1, 3, 5).reshape(B, (H // p) * (W // p), C * p * p)


class FluxPipeline(TrainingPipeline):
    architecture = "flux"

    def _objective(self):
        c = self.config
        return FlowMatching(c.timestep_sampler, {})

    def sample_timesteps(self, n, gen=None, device="cpu", seq_len=None):
        t = super().sample_timesteps(n, gen, device)
        if self.config.dynamic_shift and seq_len is not None:
            # shift = lerp(0.5, 1.15) over 256..4096 image tokens; t' = t + shift * t (1 - t)
            # (crates/training/src/pipelines/flux_pipeline.rs:185-216)
            f = min(max((seq_len - 256) / (4096 - 256), 0.0), 1.0)
            shift = 0.5 + (1.15 - 0.5) * f
            t = (t + shift * t * (1 - t)).clamp(0, 1)
        return t

    def pack(self, x):
        return _patchify(x, self.config.patch)

    def get_model_inputs(self, noisy, t, prompt, batch):
        B = noisy.shape[0]
        H, W = noisy.shape[-2] // self.config.patch, noisy.shape[-1] // self.config.patch
        return dict(img=self.pack(noisy), txt=prompt.encoder_hidden_states, t=t, y=prompt.pooled_projections,
                    guidance=torch.full((B,), float(self.config.guidance), device=noisy.device), grid_hw=(H, W))

    def call_model(self, model, inputs):
        if not getattr(getattr(model, "cfg", None), "guidance_embed", False):
            inputs = {**inputs, "guidance": None}
        return model(inputs["img"], inputs["txt"], inputs["t"], inputs["y"], inputs["guidance"], grid_hw=inputs["grid_hw"])

    def training_loss(self, model, batch, gen=None):
        pb = self.prepare_batch(batch)
        p = self.config.patch
        seq = (pb.latents.shape[-2] // p) * (pb.latents.shape[-1] // p)
        t = self.sample_timesteps(pb.latents.shape[0], gen, pb.latents.device, seq_len=seq)
        noisy, target = self.add_noise(pb.latents, self.make_noise(pb.latents, gen), t)
        return self.compute_loss(model, noisy, target, t, pb.prompt, pb)


class SD3Pipeline(FluxPipeline):
    architecture = "sd3"

    def _objective(self):
        return FlowMatching(self.config.timestep_sampler, {}, "snr_sqrt" if self.config.snr_sqrt_weighting else "none")

    def sample_timesteps(self, n, gen=None, device="cpu", seq_len=None):
        return TrainingPipeline.sample_timesteps(self, n, gen, device)

    @staticmethod
    def combine_text(clip_l, clip_g, t5, pooled_l, pooled_g):
        """CLIP-L (768) and CLIP-G (1280) hidden states are concatenated on the feature axis and
        zero-padded to the T5 width, then joined with T5 on the token axis; pooled = [L | G] = 2048
        (crates/training/src/sd35_trainer_impl.rs:53-101)."""
        clip = torch.cat([clip_l, clip_g], dim=-1)
        clip = torch.nn.functional.pad(clip, (0, t5.shape[-1] - clip.shape[-1]))
        return PromptEmbeds(torch.cat([clip, t5], dim=1), torch.cat([pooled_l, pooled_g], dim=-1))

    def call_model(self, model, inputs):
        return model(inputs["img"], inputs["txt"], inputs["t"], inputs["y"], None, grid_hw=inputs["grid_hw"])


class SDXLPipeline(TrainingPipeline):
    architecture = "sdxl"

    def _objective(self):
        c = self.config
        return DDPM(prediction=c.prediction_type, zero_terminal_snr=c.zero_terminal_snr, min_snr_gamma=c.min_snr_gamma)

    @staticmethod
    def time_ids(orig_hw, crop_yx, target_hw, batch, device="cpu"):
        return torch.tensor([[*orig_hw, *crop_yx, *target_hw]] * batch, dtype=torch.float32, device=device)

    def get_model_inputs(self, noisy, t, prompt, batch):
        B = noisy.shape[0]
        ids = batch.extras.get("time_ids")
        if ids is None:
            H, W = noisy.shape[-2] * 8, noisy.shape[-1] * 8
            ids = self.time_ids((H, W), (0, 0), (H, W), B, noisy.device)
        return dict(x=noisy, t=t, ctx=prompt.encoder_hidden_states, pooled=prompt.pooled_projections, time_ids=ids)


class SD15Pipeline(SDXLPipeline):
    architecture = "sd15"

    def get_model_inputs(self, noisy, t, prompt, batch):
        return dict(x=noisy, t=t, ctx=prompt.encoder_hidden_states)


class LTXPipeline(TrainingPipeline):
    architecture = "ltx"

    def _objective(self):
        return FlowMatching(self.config.timestep_sampler, {})

    def get_model_inputs(self, noisy, t, prompt, batch):
        # token-major latents [B, C, L, 1]
        return dict(x=noisy.squeeze(-1).transpose(1, 2), ctx=prompt.encoder_hidden_states, t=t,
                    grid_fhw=batch.extras["grid_fhw"])

    def pack(self, x):
        return x.squeeze(-1).transpose(1, 2)


class PipelineFactory:
    _KINDS = {"flux": FluxPipeline, "chroma": FluxPipeline, "krea": FluxPipeline, "qwen_image": FluxPipeline,
              "tiny_mmdit": FluxPipeline, "sd3": SD3Pipeline, "sd35": SD3Pipeline, "sdxl": SDXLPipeline,
              "sd15": SD15Pipeline, "ltx": LTXPipeline, "ltx_video": LTXPipeline}

    @classmethod
    def create(cls, architecture: str, config: PipelineConfig | None = None) -> TrainingPipeline:
        try:
            return cls._KINDS[architecture](config)
        except KeyError:
            raise ValueError(f"no training pipeline for architecture {architecture!r}; known: {sorted(cls._KINDS)}")

    @classmethod
    def known(cls):
        return sorted(cls._KINDS)


# ---------------------------------------------------------------------------- staged executor
class StageName(str, enum.Enum):
    SEED = "seed"
    FETCH_BATCH = "fetch_batch"
    TEXT_ENCODE = "text_encode"
    VAE_ENCODE = "vae_encode"
    NOISE_SCHEDULE = "noise_schedule"
    FORWARD = "forward"
    LOSS = "loss"
    BACKWARD = "backward"
    OPTIM_STEP = "optim_step"
    ZERO_GRAD = "zero_grad"
    EMA_UPDATE = "ema_update"
    CHECKPOINT = "checkpoint"
    EVAL_STEP = "eval_step"


@dataclass
class Ctx:
    step: int = 0
    rng_seed: int = 0
    batch: dict | None = None
    prepared: PreparedBatch | None = None
    noise: torch.Tensor | None = None
    timestep: torch.Tensor | None = None
    noisy: torch.Tensor | None = None
    target: torch.Tensor | None = None
    pred: torch.Tensor | None = None
    loss: torch.Tensor | None = None
    gen: torch.Generator | None = None
    log: list = field(default_factory=list)


DEFAULT_RECIPE = (StageName.SEED, StageName.FETCH_BATCH, StageName.NOISE_SCHEDULE, StageName.FORWARD, StageName.LOSS,
                  StageName.BACKWARD, StageName.OPTIM_STEP, StageName.ZERO_GRAD, StageName.EMA_UPDATE)


class PipelineAdapter:
    """Runs one stage at a time over a model, a ``TrainingPipeline``, an optimizer and a batch
    iterator (the reference's ``ModelAdapter::run(stage, cfg, ctx)``)."""

    def __init__(self, model, pipeline: TrainingPipeline, optimizer, batches, ema=None, max_grad_norm=0.0,
                 text_encoder=None, vae=None, checkpoint_fn=None, eval_fn=None):
        self.model, self.pipeline, self.optimizer, self.batches = model, pipeline, optimizer, iter(batches)
        self.ema, self.max_grad_norm = ema, max_grad_norm
        self.text_encoder, self.vae, self.checkpoint_fn, self.eval_fn = text_encoder, vae, checkpoint_fn, eval_fn

    def default_recipe(self):
        return DEFAULT_RECIPE

    def run(self, stage: StageName, ctx: Ctx):
        p = self.pipeline
        ctx.log.append(stage)
        if stage == StageName.SEED:
            ctx.gen = torch.Generator().manual_seed(ctx.rng_seed * 1000003 + ctx.step)
        elif stage == StageName.FETCH_BATCH:
            ctx.batch = next(self.batches)
            ctx.prepared = p.prepare_batch(ctx.batch) if "txt" in ctx.batch and "latents" in ctx.batch else None
        elif stage == StageName.TEXT_ENCODE:
            if "txt" not in ctx.batch:
                e = p.encode_prompts(ctx.batch["captions"], self.text_encoder)
                ctx.batch = {**ctx.batch, "txt": e.encoder_hidden_states,
                             **({"pooled": e.pooled_projections} if e.pooled_projections is not None else {})}
        elif stage == StageName.VAE_ENCODE:
            if "latents" not in ctx.batch:
                ctx.batch = {**ctx.batch, "latents": p.encode_images(ctx.batch["images"], self.vae)}
        elif stage == StageName.NOISE_SCHEDULE:
            if ctx.prepared is None:
                ctx.prepared = p.prepare_batch(ctx.batch)
            x0 = ctx.prepared.latents
            ctx.timestep = p.sample_timesteps(x0.shape[0], ctx.gen, x0.device)
            ctx.noise = p.make_noise(x0, ctx.gen)
            ctx.noisy, ctx.target = p.add_noise(x0, ctx.noise, ctx.timestep)
        elif stage == StageName.FORWARD:
            pb = ctx.prepared
            ctx.pred = p.postprocess_outputs(p.call_model(self.model, p.get_model_inputs(ctx.noisy, ctx.timestep,
                                                                                        pb.prompt, pb)), pb)
        elif stage == StageName.LOSS:
            ctx.loss = loss_fn(p.config.loss, ctx.pred, p.pack(ctx.target), p.apply_snr_weight(ctx.timestep))
        elif stage == StageName.BACKWARD:
            ctx.loss.backward()
        elif stage == StageName.OPTIM_STEP:
            if self.max_grad_norm > 0:
                torch.nn.utils.clip_grad_norm_([q for g in self.optimizer.param_groups for q in g["params"]],
                                               self.max_grad_norm)
            self.optimizer.step()
        elif stage == StageName.ZERO_GRAD:
            self.optimizer.zero_grad(set_to_none=True)
        elif stage == StageName.EMA_UPDATE:
            if self.ema is not None:
                self.ema.update()
        elif stage == StageName.CHECKPOINT:
            if self.checkpoint_fn is not None:
                self.checkpoint_fn(ctx.step)
        elif stage == StageName.EVAL_STEP:
            if self.eval_fn is not None:
                self.eval_fn(ctx.step)
        else:
            raise ValueError(stage)


class Orchestrator:
    def __init__(self, adapter: PipelineAdapter, recipe=None):
        self.adapter = adapter
        self.recipe = [StageName(s) for s in (recipe or adapter.default_recipe())]

    def run_step(self, ctx: Ctx) -> Ctx:
        for stage in self.recipe:
            self.adapter.run(stage, ctx)
        ctx.step += 1
        return ctx
