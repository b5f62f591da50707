"""Small applications built on the runtime and the function library, the counterparts of the reference's
``examples/`` programs that carry logic of their own: a streaming voice-activity detector and the samplers of a
latent-diffusion pipeline."""
