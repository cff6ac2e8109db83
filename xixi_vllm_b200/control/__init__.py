"""Control plane: facade, clients, engine core, scheduler, executors."""
