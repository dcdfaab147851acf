//! rstorch's training-step API on B200 GPUs.
//!
//! The crate keeps the names and signatures of `rstorch` 0.2.0 for the training step
//! (`sequential!`, `Module::{forward, backward, parameters}`, `CrossEntropyLoss`,
//! `SGD::new(lr).step(&mut model)`, `DataLoader::iter_array`, `accuracy`) and routes them
//! through the C ABI of `librstorch_b200.so`.  The one change a caller sees is the matrix
//! type: the device [`Tensor`] where the reference passes `Array2<f64>`; `Tensor::from(array)`
//! and `Tensor::to_array()` convert at the edges.  There is no CPU path: without the library
//! and a GPU every constructor panics.
//!
//! ```ignore
//! use rstorch_b200::prelude::*;
//! use rstorch_b200::utils::accuracy;
//! use rstorch_b200::{CrossEntropyLoss, Identity, Linear, ReLU, SGD};
//!
//! let mut model = sequential!(Identity(), Linear(784, 100), ReLU(), Linear(100, 100), ReLU(), Linear(100, 10));
//! let mut loss = CrossEntropyLoss::new();
//! let mut optim = SGD::new(0.01);
//! for (x, y) in data_loader.iter_array() {
//!     let pred = model.forward(x);
//!     let l = loss.forward(pred.clone(), y.clone());
//!     let acc = accuracy(pred, y);
//!     model.backward(loss.backward());
//!     optim.step(&mut model);
//! }
//! ```
pub mod data;
pub mod dataset;
pub mod ffi;
pub mod graph;
pub mod loss;
pub mod model;
pub mod module;
pub mod optim;
pub mod parallel;
pub mod tensor;
pub mod utils;

pub use dataset::DeviceDataset;
pub use graph::Graph;
pub use loss::CrossEntropyLoss;
pub use model::BasicModel;
pub use module::{Identity, Linear, ReLU, Sequential, Softmax};
pub use optim::SGD;
pub use tensor::{Context, Tensor};

pub mod prelude {
    // traits
    pub use crate::data::{Dataset, Sampler};
    pub use crate::loss::Loss;
    pub use crate::module::init::InitParameters;
    pub use crate::module::Module;
    pub use crate::optim::Optimizer;

    // types the README loop names through the prelude
    pub use crate::data::{DataLoader, SequentialSampler};
    pub use crate::tensor::{Context, Tensor};

    // macros
    pub use crate::sequential;

    pub use ndarray::prelude::*;
}
