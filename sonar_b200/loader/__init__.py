from sonar_b200.loader.weights import load_model, save_checkpoint  # noqa: F401
