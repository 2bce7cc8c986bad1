"""The step function, the model on its device, and the generation loop."""
